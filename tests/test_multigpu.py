"""Real multi-GPU runs (NVLink / NVSwitch, NVLS when present): spawns
tests/mgpu_worker.py with one process per GPU."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(nproc: int, script: str, *args, timeout=600):
    port = 29500 + (os.getpid() % 1000)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, script), *args]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)


@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_collectives_on_real_gpus(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    r = _run(nproc, "mgpu_worker.py")
    tail = (r.stdout + r.stderr)[-4000:]
    assert r.returncode == 0, tail
    line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
    res = json.loads(line)
    assert res["total_failures"] == 0 and res["cases"] > 20, tail
