"""Per-tile timeline of the fused GEMM kernels on real GPUs: every CTA stamps
%globaltimer when its producer may load a tile, when the tile's accumulator is
complete and when its epilogue is done, plus (CTA-pair kernels) the phases around
the mainloop: data-mover batches stored / acknowledged, mainloop left, first wait
of the final reduction over, kernel left, reduction units done between tiles and
at the end.  Rank 0 prints its own per-tile table and one summary line per rank
(every rank's times are relative to ITS first CTA: the GPUs' timers are not
synchronised) — the numbers that say whether a kernel is MMA-, link-, arrival-
or skew-bound.  ncu cannot show this: it never wraps a multi-rank command.

    python -m torch.distributed.run --nproc-per-node 8 bench/trace_fused.py [--variant pair|single]
        [--movers-only 1]     # all-gather -> GEMM: move the shard, compute nothing (pair kernel)
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


def _us(t, col, start):
    v = t[:, col]
    m = v > 0
    if not bool(m.any()):
        return None
    d = (v[m] - start).double() / 1e3  # int64 arithmetic first: the timer is ~1e17 ns
    return float(d.mean()), float(d.max())


def per_tile(name, t):
    start = int(t[:, 63].min())
    us = lambda x: (x - start).double() / 1e3
    print(f"--- {name}, rank 0: {t.shape[0]} CTAs; kernel start skew between CTAs {float(us(t[:, 63]).max()):.1f} us")
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


def per_rank(name, traces, labels, counters=None):
    """One line per rank: mean / max over its CTAs of every phase stamp in `labels` {word: text};
    `counters` {word: text} are summed over the CTAs."""
    for r, t in enumerate(traces):
        start = int(t[:, 63].min())
        parts = []
        for col, text in labels.items():
            v = _us(t, col, start)
            if v:
                parts.append(f"{text} {v[0]:.1f}/{v[1]:.1f}")
        for col, text in (counters or {}).items():
            parts.append(f"{text} {int(t[:, col].sum())}")
        done = t[:, 2:56:4]
        last = float((done.max() - start)) / 1e3 if bool((done > 0).any()) else 0.0
        parts.append(f"last epilogue {last:.1f}")
        print(f"  {name} rank {r}: " + " | ".join(parts) + "  (mean/max us)")


def gather(tr, grid, W, rank):
    t = tr.view(grid, 64)
    if W == 1:
        return [t.cpu()]
    bufs = [torch.empty_like(t) for _ in range(W)] if rank == 0 else None
    dist.gather(t, bufs, dst=0)
    return [b.cpu() for b in bufs] if rank == 0 else None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--variant", default="pair", choices=["pair", "single"])
    ap.add_argument("--movers-only", type=int, default=0)
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
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    a_r, wd_r = rnd((T, Il), 4000 + rank), rnd((H, Il), 5000 + rank, 0.02)
    for it in range(5):
        tr.zero_()
        dist.barrier()
        flush.zero_()  # the kernel queues behind this on every rank: launches skew less than after a host barrier
        tccl.gemm_reduce_scatter(a_r, wd_r, trace=tr, variant=a.variant)
        torch.cuda.synchronize()
    ts = gather(tr, grid, W, rank)
    if rank == 0:
        per_tile("gemm_reduce_scatter", ts[0])
        per_rank("gemm_rs", ts, {60: "mainloop left", 59: "first final wait over", 61: "leave"},
                 {58: "units reduced between tiles", 57: "units reduced at the end"})
    x_sh, wu_r = rnd((rows, H), 4000 + rank), rnd((Il, H), 6000 + rank, 0.02)
    movers = 2 if (a.movers_only and a.variant == "pair") else False
    for it in range(5):
        tr.zero_()
        dist.barrier()
        flush.zero_()
        tccl.all_gather_gemm(x_sh, wu_r, trace=tr, variant=a.variant, lsu_movers=movers)
        torch.cuda.synchronize()
    ts = gather(tr, grid, W, rank)
    if rank == 0:
        t0 = ts[0] if a.variant == "pair" else ts[0][w.config.ag_movers:]
        per_tile("all_gather_gemm" + (" (movers only)" if movers else ""), t0)
        per_rank("ag_gemm", ts, {60: "batch 0 stored", 59: "batch 0 acknowledged", 58: "batch 1 stored",
                                 57: "batch 1 acknowledged", 62: "movers done", 61: "leave"})
    w.check()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
