"""Small single-GPU workloads for `ncu` captures (one kernel, a few launches,
inputs larger than L2 but far below a GB):

    python bench/profile_targets.py gemm --m 4096 --n 4096 --k 1792 --iters 4
    python bench/profile_targets.py copy --mib 256 --iters 4        # one-rank all-reduce = local copy
    python bench/profile_targets.py emu_allreduce --world 4 --mib 64 --algo twoshot_p2p --iters 4
    python bench/profile_targets.py emu_gemm_rs --world 2 --iters 3
    python bench/profile_targets.py emu_rmsnorm --world 4 --iters 4

Each prints the CUDA-event time of its last iteration so that the same command
line can first be run plainly (exit code 0) and then under ncu.
"""
import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import tccl_b200 as tccl  # noqa: E402
from tccl_b200.config import Config  # noqa: E402
from tccl_b200.parallel.emu import EmuWorld  # noqa: E402


def timed(fn, iters):
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    for i in range(iters):
        if i == iters - 1:
            ev[0].record()
        fn()
    ev[1].record()
    torch.cuda.synchronize()
    return ev[0].elapsed_time(ev[1]) * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "copy", "emu_allreduce", "emu_gemm_rs", "emu_ag_gemm", "emu_rmsnorm",
                                     "emu_tree"])
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=1792)
    ap.add_argument("--mib", type=int, default=256)
    ap.add_argument("--world", type=int, default=4)
    ap.add_argument("--algo", default="twoshot_p2p")
    ap.add_argument("--iters", type=int, default=4)
    a = ap.parse_args()
    dev = "cuda"
    cfg = Config.from_env()
    cfg.stage_mb = 64
    rnd = lambda *s, sc=1.0: (torch.randn(*s, device=dev) * sc).to(torch.bfloat16)
    if a.what == "gemm":
        x, wt = rnd(a.m, a.k), rnd(a.n, a.k, sc=0.02)
        out = torch.empty(a.m, a.n, dtype=torch.bfloat16, device=dev)
        us = timed(lambda: tccl.gemm_bf16(x, wt, out=out), a.iters)
        print(f"gemm {a.m}x{a.n}x{a.k}: {us:.1f} us, {2.0 * a.m * a.n * a.k / us / 1e6:.0f} TFLOP/s")
    elif a.what == "copy":
        w = EmuWorld(1, config=cfg)
        n = a.mib << 19
        x = w.from_parts([rnd(n)])
        out = [torch.empty(n, dtype=torch.bfloat16, device=dev)]
        from tccl_b200.parallel.emu import EmuTensor
        o = EmuTensor(out)
        us = timed(lambda: tccl.all_reduce(x, out=o, algo="oneshot_p2p", world=w), a.iters)
        print(f"copy {a.mib} MiB: {us:.1f} us, {2.0 * n * 2 / us / 1e3:.0f} GB/s read+write")
    elif a.what in ("emu_allreduce", "emu_tree"):
        w = EmuWorld(a.world, config=cfg)
        n = a.mib << 19
        x = w.from_parts([rnd(n) for _ in range(a.world)])
        algo = "tree" if a.what == "emu_tree" else a.algo
        if algo.startswith("oneshot"):
            fn = lambda: tccl.all_reduce(x, algo=algo, world=w)
        else:
            fn = lambda: tccl.all_reduce(x, inplace=True, algo=algo, world=w)
        us = timed(fn, a.iters)
        w.check()
        print(f"emulated {algo} W={a.world} {a.mib} MiB: {us:.1f} us")
    elif a.what == "emu_gemm_rs":
        w = EmuWorld(a.world, config=cfg)
        A = [rnd(a.m, a.k) for _ in range(a.world)]
        B = [rnd(a.n, a.k, sc=0.02) for _ in range(a.world)]
        us = timed(lambda: tccl.gemm_reduce_scatter(A, B, world=w), a.iters)
        w.check()
        print(f"emulated gemm_rs W={a.world} {a.m}x{a.n}x{a.k}: {us:.1f} us")
    elif a.what == "emu_ag_gemm":
        w = EmuWorld(a.world, config=cfg)
        A = [rnd(a.m // a.world, a.k) for _ in range(a.world)]
        B = [rnd(a.n, a.k, sc=0.02) for _ in range(a.world)]
        us = timed(lambda: tccl.all_gather_gemm(A, B, world=w), a.iters)
        w.check()
        print(f"emulated ag_gemm W={a.world} {a.m}x{a.n}x{a.k}: {us:.1f} us")
    elif a.what == "emu_rmsnorm":
        w = EmuWorld(a.world, config=cfg)
        T, H = a.m, a.n
        x = w.from_parts([rnd(T, H) for _ in range(a.world)])
        wn, b, r = rnd(H), rnd(H), rnd(T, H)
        rep = lambda t: [t] * a.world
        us = timed(lambda: tccl.all_reduce_bias_residual_rmsnorm(x, rep(wn), rep(b), rep(r), world=w), a.iters)
        w.check()
        print(f"emulated allreduce+rmsnorm W={a.world} {T}x{H}: {us:.1f} us")


if __name__ == "__main__":
    main()
