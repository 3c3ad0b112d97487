"""Per-tile timeline of the fused GEMM kernels on real GPUs: every CTA stamps
%globaltimer when its producer may load a tile, when the tile's accumulator is
complete and when its epilogue is done (plus, in the CTA-pair kernels, when the
epilogue warps are through with their data-mover phase and when the CTA leaves).
Prints, for rank 0, the kernel span and the distribution of epilogue durations
and of the producer's wait per tile position — the numbers that say whether the
kernel is MMA-, link- or arrival-bound.  ncu cannot show this: it never wraps a
multi-rank command.

    python -m torch.distributed.run --nproc-per-node 8 bench/trace_fused.py [--variant pair|single]
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import tccl_b200 as tccl  # noqa: E402


def rnd(shape, seed, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).cuda()


def summarize(name, tr, grid, comm_ctas=0):
    t = tr.view(grid, 64).cpu()[comm_ctas:]
    start = int(t[:, 63].min())
    us = lambda x: (x - start).double() / 1e3  # int64 arithmetic first: the timer is ~1e17 ns
    print(f"--- {name}: {t.shape[0]} GEMM CTAs; kernel start skew {float(us(t[:, 63]).max()):.1f} us")
    if bool((t[:, 62] > 0).any()):
        m = t[:, 62] > 0
        print(f"  epilogue warps free (data-mover phase over) at: mean {float(us(t[:, 62][m]).mean()):.1f} max "
              f"{float(us(t[:, 62][m]).max()):.1f} us")
    if bool((t[:, 61] > 0).any()):
        m = t[:, 61] > 0
        print(f"  CTAs leave at: mean {float(us(t[:, 61][m]).mean()):.1f} max {float(us(t[:, 61][m]).max()):.1f} us")
    last = 0.0
    for i in range(8):
        load, ready, done = t[:, 4 * i], t[:, 4 * i + 1], t[:, 4 * i + 2]
        m = done > 0
        if not bool(m.any()):
            break
        l, r, d = us(load[m]), us(ready[m]), us(done[m])
        last = max(last, float(d.max()))
        print(f"  tile #{i}: CTAs {int(m.sum()):3d} | may load: mean {float(l.mean()):6.1f} max {float(l.max()):6.1f} us"
              f" | acc ready: mean {float(r.mean()):6.1f} us | epilogue done: mean {float(d.mean()):6.1f} max "
              f"{float(d.max()):6.1f} us | epilogue takes mean {float((d - r).mean()):5.1f} max {float((d - r).max()):5.1f} us")
    print(f"  last epilogue done at {last:.1f} us after the first CTA started")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--variant", default="pair", choices=["pair", "single"])
    a = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    W = int(os.environ.get("WORLD_SIZE", 1))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29545")
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", rank=rank, world_size=W, device_id=torch.device("cuda", local_rank))
    w = tccl.init()
    T, H, I = 4096, 4096, 14336
    Il, rows = I // W, T // W
    grid = w.num_sms() & ~1 if a.variant == "pair" else w.num_sms()
    tr = torch.zeros(grid * 64, dtype=torch.int64, device="cuda")
    a_r, wd_r = rnd((T, Il), 4000 + rank), rnd((H, Il), 5000 + rank, 0.02)
    for it in range(4):
        tr.zero_()
        dist.barrier()
        tccl.gemm_reduce_scatter(a_r, wd_r, trace=tr, variant=a.variant)
        torch.cuda.synchronize()
    if rank == 0:
        summarize("gemm_reduce_scatter", tr, grid)
    x_sh, wu_r = rnd((rows, H), 4000 + rank), rnd((Il, H), 6000 + rank, 0.02)
    for it in range(4):
        tr.zero_()
        dist.barrier()
        tccl.all_gather_gemm(x_sh, wu_r, trace=tr, variant=a.variant)
        torch.cuda.synchronize()
    if rank == 0:
        summarize("all_gather_gemm", tr, grid, comm_ctas=0 if a.variant == "pair" else w.config.ag_movers)
    w.check()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
