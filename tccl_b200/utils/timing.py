"""Device-side timing: CUDA events around every iteration on the launching
stream, after warm-up, synchronised on both sides; multi-rank numbers are the
per-iteration maximum over ranks."""
from __future__ import annotations

import statistics
from typing import Callable, List, Optional

import torch


class L2Flusher:
    """Writes a buffer larger than the 126 MB L2 so the next kernel starts cold."""

    def __init__(self, device, nbytes: int = 256 << 20):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)

    def __call__(self):
        self.buf.zero_()


def time_iters(fn: Callable[[], None], iters: int, warmup: int, *, before: Optional[Callable[[], None]] = None,
               sync: Optional[Callable[[], None]] = None) -> List[float]:
    """Milliseconds of every timed iteration of ``fn`` (one entry per iteration).
    ``before`` runs untimed ahead of each iteration (L2 flush, input refresh);
    ``sync`` is a cross-rank barrier called next to the device synchronise."""
    for _ in range(warmup):
        if before:
            before()
        fn()
    torch.cuda.synchronize()
    if sync:
        sync()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    for i in range(iters):
        if before:
            before()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    if sync:
        sync()
    return [s.elapsed_time(e) for s, e in zip(starts, ends)]


def max_over_ranks(ms: List[float], group=None) -> List[float]:
    """Per-iteration maximum over the ranks of ``group`` (no-op without c10d)."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return ms
    t = torch.tensor(ms, dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t.cpu().tolist()


def summarize(ms: List[float]) -> dict:
    s = sorted(ms)
    q = lambda f: s[min(len(s) - 1, int(f * len(s)))]
    return {"p50_us": statistics.median(s) * 1e3, "p10_us": q(0.10) * 1e3, "p90_us": q(0.90) * 1e3,
            "min_us": s[0] * 1e3, "mean_us": statistics.fmean(s) * 1e3, "iters": len(s)}
