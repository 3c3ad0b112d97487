"""The TCCL_DEBUG_CHECKS flavour of the library: the flat collectives check every vector offset
against the extents the host passes; a miss is recorded as TCCL_BAD_INDEX and the access is skipped.

The flavour is chosen when the package is imported (environment variable), so the checks run in a
child process.  The "miss" is produced on the host: the wrapper is told to claim 32 bytes less input
than there is (``debug_shrink_extent``), so the kernel's own arithmetic steps over the claimed extent
while every address it would have touched is still inside the real buffer."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import json, sys, torch
sys.path.insert(0, %r)
import tccl_b200 as tccl
from tccl_b200.config import Config
from tccl_b200.parallel.emu import EmuWorld
from tccl_b200.utils import lib as L

res = {"flavour": int(L.lib().tccl_debug_checks())}
cfg = Config(); cfg.stage_mb = 8; cfg.tree_ctas = 2; cfg.timeout_ms = 2000.0
W, n = 4, 4096 + 8
w = EmuWorld(W, config=cfg)
parts = [torch.randn(n, generator=torch.Generator().manual_seed(r)).to(torch.bfloat16) for r in range(W)]
x = w.from_parts(parts)
ref = torch.stack([p.float() for p in x.parts]).sum(0)
ok = lambda o, r: bool(((o.float() - r).abs() <= r.abs() * 2 ** -8 + 1e-5).all())
good = True
for algo in ("oneshot_p2p", "push_p2p"):
    out = tccl.all_reduce(x, algo=algo, world=w)
    torch.cuda.synchronize()
    good = good and all(ok(out[r], ref) for r in range(W))
for algo in ("twoshot_p2p", "twoshot_pipe_p2p"):
    y = w.from_parts([p.clone() for p in parts])
    tccl.all_reduce(y, inplace=True, algo=algo, world=w)
    torch.cuda.synchronize()
    good = good and all(ok(y[r], ref) for r in range(W))
g = tccl.all_gather(x, algo="pull", world=w)
og = w.empty((W, n), torch.bfloat16)
tccl.all_gather(x, out=og, algo="push", world=w)
z = w.from_parts([p[: 4096].clone() for p in parts])
rs = tccl.reduce_scatter(z, world=w)
torch.cuda.synchronize()
full = torch.stack(list(x.parts))
good = good and all(torch.equal(g[r], full) and torch.equal(og[r], full) for r in range(W))
good = good and all(ok(rs[r], ref[:4096].view(W, -1)[r]) for r in range(W))
res["clean_results_ok"] = good
res["clean_status"] = [s["code"] for s in w.last_status()]
# now claim 32 bytes less input than there is: the last two vectors are beyond the claimed extent
w.config.debug_shrink_extent = 32
tccl.all_reduce(x, algo="oneshot_p2p", world=w)
torch.cuda.synchronize()
st = w.last_status(0)
res["shrunk_status"] = {k: st[k] for k in ("code", "where", "seen", "want")}
w.reset()
w.config.debug_shrink_extent = 0
out = tccl.all_reduce(x, algo="oneshot_p2p", world=w)
torch.cuda.synchronize()
res["after_reset_ok"] = all(ok(out[r], ref) for r in range(W)) and all(s["code"] == 0 for s in w.last_status())
print("RESULT " + json.dumps(res))
""" % ROOT


def _run(env_extra):
    env = dict(os.environ)
    env.update(env_extra)
    r = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, timeout=600, env=env)
    lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
    assert r.returncode == 0 and lines, (r.stdout[-2000:], r.stderr[-3000:])
    return json.loads(lines[-1][7:])


def test_debug_flavour_checks_every_offset_and_reports_a_miss_without_faulting():
    from tccl_b200.utils.consts import K

    res = _run({"TCCL_DEBUG_CHECKS": "1"})
    assert res["flavour"] == 1
    assert res["clean_results_ok"] and res["clean_status"] == [0, 0, 0, 0]
    st = res["shrunk_status"]
    n_bytes = (4096 + 8) * 2
    assert st["code"] == K["TCCL_BAD_INDEX"] and st["where"] == "TCCL_W_INDEX_IN"
    assert st["want"] == n_bytes - 32 and n_bytes - 32 <= st["seen"] < n_bytes  # the offending offset, the claimed extent
    assert res["after_reset_ok"]


def test_regular_flavour_ignores_the_extents():
    res = _run({"TCCL_DEBUG_CHECKS": ""})
    assert res["flavour"] == 0 and res["clean_results_ok"]
    assert res["shrunk_status"]["code"] == 0 and res["after_reset_ok"]
