"""NumPy model of the pipelined double-tree all-reduce (CPU only).

This is the host-side twin of the device protocol in ``csrc/tree_allreduce.cu``:
the message is cut into chunks, chunk ``c`` travels over tree ``c % 2``; on
every rank and tree an *up worker* streams through that tree's chunks (wait
for the children's "partial ready" counters, pull the children's partials out
of their buffers, add the own data, store the partial **in place**, bump the
parent's counter; the root's result is final and it bumps its child's "final
ready" counter instead) and a *down worker* streams through the same chunks
(wait for the parent's "final ready" counter, pull the final chunk from the
parent's buffer into the own buffer, bump the children's counters).  The
workers are Python generators that ``yield`` where the kernel spins on a
flag, and a scheduler interleaves them in a seeded random order, so the model
checks the protocol (no deadlock for any interleaving it tries, no read of a
chunk before it is published) as well as the arithmetic.

The reference only describes this algorithm (``tree.py:36-51``,
``triton_double_tree_allreduce.py:254-335``); its kernel never completed it.
"""
from __future__ import annotations

import random
from typing import List, Optional, Sequence

import numpy as np

from .tree import tree_neighbours

__all__ = ["simulate_double_tree_all_reduce", "chunk_bounds"]


def chunk_bounds(numel: int, n_chunks: int, align: int = 1) -> List[tuple]:
    """Split ``[0, numel)`` into ``n_chunks`` contiguous ranges whose starts are
    multiples of ``align`` (trailing chunks may be empty)."""
    per = -(-numel // n_chunks)
    per = -(-per // align) * align
    out = []
    for c in range(n_chunks):
        lo = min(c * per, numel)
        hi = min(lo + per, numel)
        out.append((lo, hi))
    return out


class _Deadlock(RuntimeError):
    pass


def simulate_double_tree_all_reduce(
    inputs: Sequence[np.ndarray],
    n_chunks: int = 64,
    seed: Optional[int] = 0,
    acc_dtype=np.float32,
) -> List[np.ndarray]:
    """All-reduce ``inputs`` (one array per rank, same shape) over the double
    binary tree; returns one result array per rank.  ``inputs`` are not
    modified (the in-place buffers are copies)."""
    W = len(inputs)
    numel = inputs[0].size
    bufs = [np.array(x, dtype=acc_dtype, copy=True).reshape(-1) for x in inputs]
    bounds = chunk_bounds(numel, n_chunks)
    nbr = [[tree_neighbours(W, r, t) for t in (0, 1)] for r in range(W)]

    # counters, all written by a *peer* and polled by the owner (as on the GPU)
    up_cnt = [[[0, 0] for _ in range(2)] for _ in range(W)]   # [rank][tree][child slot]
    down_cnt = [[0, 0] for _ in range(W)]                      # [rank][tree]
    published = [[set() for _ in range(2)] for _ in range(W)]  # chunks whose partial is in place
    final = [[set() for _ in range(2)] for _ in range(W)]      # chunks whose final value is in place

    def chunks_of(tree):
        return [c for c in range(n_chunks) if c % 2 == tree]

    def up_worker(r, t):
        parent, left, right = nbr[r][t]
        kids = [k for k in (left, right) if k >= 0]
        for n, c in enumerate(chunks_of(t)):
            lo, hi = bounds[c]
            for slot, k in enumerate(kids):
                while up_cnt[r][t][slot] < n + 1:
                    yield
            acc = bufs[r][lo:hi].copy()
            for k in kids:
                assert c in published[k][t], "read of an unpublished partial"
                acc += bufs[k][lo:hi]
            bufs[r][lo:hi] = acc
            published[r][t].add(c)
            if parent >= 0:
                slot = [k for k in nbr[parent][t][1:] if k >= 0].index(r)
                up_cnt[parent][t][slot] += 1
            else:
                final[r][t].add(c)
                for k in kids:
                    down_cnt[k][t] += 1

    def down_worker(r, t):
        parent, left, right = nbr[r][t]
        if parent < 0:
            return
        kids = [k for k in (left, right) if k >= 0]
        for n, c in enumerate(chunks_of(t)):
            lo, hi = bounds[c]
            while down_cnt[r][t] < n + 1:
                yield
            assert c in final[parent][t], "read of a non-final chunk"
            bufs[r][lo:hi] = bufs[parent][lo:hi]
            final[r][t].add(c)
            for k in kids:
                down_cnt[k][t] += 1

    workers = []
    for r in range(W):
        for t in (0, 1):
            workers.append(up_worker(r, t))
            workers.append(down_worker(r, t))
    rng = random.Random(seed)
    idle_rounds = 0
    while workers:
        rng.shuffle(workers)
        progressed = False
        alive = []
        before = (sum(map(len, (s for p in published for s in p))),
                  sum(map(len, (s for p in final for s in p))))
        for w in workers:
            try:
                next(w)
                alive.append(w)
            except StopIteration:
                progressed = True
        after = (sum(map(len, (s for p in published for s in p))),
                 sum(map(len, (s for p in final for s in p))))
        progressed = progressed or after != before
        workers = alive
        idle_rounds = 0 if progressed else idle_rounds + 1
        if idle_rounds > 4:
            raise _Deadlock("double-tree protocol made no progress")
    return [b.reshape(inputs[0].shape) for b in bufs]
