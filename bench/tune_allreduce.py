"""Shape sweep of the large-message all-reduce kernels on real GPUs.

    python -m torch.distributed.run --nproc-per-node 8 bench/tune_allreduce.py \
        --mib 512,64 --out results/tune8.jsonl

For every message size it times, with the same harness as bench/sweep.py
(CUDA events per iteration, per-iteration maximum over ranks, p50):

* the plain two-shot kernel (NVLS when there is a switch, else P2P) for several CTA counts,
* the pipelined two-shot kernel (reducer / broadcaster warps, ``allreduce_pipe.cu``) over a
  grid of CTA counts, reducer warps, stages and vectors per reducer thread,
* NCCL's all-reduce.

Every configuration is checked once against the plain kernel's result before
it is timed.  One JSON line per measurement; the best pipelined shape per size
is repeated at the end with ``"best": true`` — those are the numbers the
defaults in ``tccl_b200/config.py`` come from.
"""
import argparse
import itertools
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import tccl_b200 as tccl  # noqa: E402
from tccl_b200.utils.timing import max_over_ranks, summarize, time_iters  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mib", default="512,64")
    ap.add_argument("--iters", type=int, default=12)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--ctas", default="8,16,32,64")
    ap.add_argument("--reducers", default="4,8,12")
    ap.add_argument("--stages", default="4,8")
    ap.add_argument("--unroll", default="2,4,8")
    ap.add_argument("--plain-ctas", default="4,8,16,32")
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    W = int(os.environ.get("WORLD_SIZE", 1))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29555")
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", rank=rank, world_size=W, device_id=torch.device("cuda", local_rank))
    w = tccl.init()
    nvls = w.has_nvls and W > 2
    suffix = "nvls" if nvls else "p2p"
    ints = lambda s: [int(v) for v in s.split(",") if v]
    sizes = [m << 20 for m in ints(a.mib)]
    nmax = max(sizes) // 2
    g = torch.Generator(device="cpu").manual_seed(2000 + rank)
    host = torch.randn(1 << 22, generator=g).to(torch.bfloat16)
    x = w.empty(nmax, torch.bfloat16)
    y = w.empty(nmax, torch.bfloat16)
    yref = torch.empty(min(nmax, 1 << 24), dtype=torch.bfloat16, device="cuda")
    for off in range(0, nmax, host.numel()):
        m = min(host.numel(), nmax - off)
        x[off:off + m].copy_(host[:m])
    rows = []

    def emit(r):
        rows.append(r)
        if rank == 0:
            print(json.dumps(r), flush=True)

    def measure(fn):
        st = summarize(max_over_ranks(time_iters(fn, a.iters, a.warmup, sync=dist.barrier)))
        w.check()
        return st["p50_us"]

    for S in sizes:
        n = S // 2
        xs, ys = x[:n], y[:n]
        m = min(n, yref.numel())
        # reference result: the plain kernel with its default grid
        w.reconfigure(max_ctas=0, pipe_min_bytes=0)
        tccl.all_reduce(xs, out=ys, algo="twoshot_" + suffix)
        torch.cuda.synchronize()
        yref[:m].copy_(ys[n - m:n])
        for c in ints(a.plain_ctas):
            w.reconfigure(max_ctas=c)
            us = measure(lambda: tccl.all_reduce(xs, out=ys, algo="twoshot_" + suffix))
            emit({"kernel": "twoshot_" + suffix, "world": W, "bytes": S, "ctas": c, "p50_us": round(us, 1),
                  "algbw_gbs": round(S / us / 1e3, 1)})
        w.reconfigure(max_ctas=0)
        best = None
        for c, nr, st, ur in itertools.product(ints(a.ctas), ints(a.reducers), ints(a.stages), ints(a.unroll)):
            if st * nr * 32 * ur * 16 > 200 * 1024:
                continue
            if not nvls and W * ur > 32:
                continue
            w.reconfigure(pipe_ctas=c, pipe_reducers=nr, pipe_stages=st, pipe_unroll=ur)
            ys.zero_()
            tccl.all_reduce(xs, out=ys, algo="twoshot_pipe_" + suffix)
            torch.cuda.synchronize()
            ok = bool(torch.equal(ys[n - m:n], yref[:m])) if nvls else bool(
                ((ys[n - m:n].float() - yref[:m].float()).abs() <= yref[:m].float().abs() * 2 ** -7 + 1e-3).all())
            us = measure(lambda: tccl.all_reduce(xs, out=ys, algo="twoshot_pipe_" + suffix))
            r = {"kernel": "twoshot_pipe_" + suffix, "world": W, "bytes": S, "ctas": c, "reducers": nr, "stages": st,
                 "unroll": ur, "p50_us": round(us, 1), "algbw_gbs": round(S / us / 1e3, 1), "verified": ok}
            emit(r)
            if ok and (best is None or us < best["p50_us"]):
                best = r
        if best:
            emit({**best, "best": True})
        ys.zero_()
        us = measure(lambda: dist.all_reduce(ys))
        emit({"kernel": "nccl", "world": W, "bytes": S, "p50_us": round(us, 1), "algbw_gbs": round(S / us / 1e3, 1)})
    if a.out and rank == 0:
        os.makedirs(os.path.dirname(a.out) or ".", exist_ok=True)
        with open(a.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
