"""NumPy model of the pipelined double-tree all-reduce (CPU only).

This is the host-side twin of the device protocol in ``csrc/tree_allreduce.cu``:
the message is cut into chunks, chunk ``c`` travels over tree ``c % 2``; on
every rank and tree an *up worker* streams through that tree's chunks — wait
for the children's UP counters (their partials sit in this rank's ring) and,
below the root, for the parent's ACK counter (the ring slot to be filled is
free again), add the own input to the ring slots, **store the partial into the
parent's ring** (slot ``[tree][child slot][n mod depth]``) and bump the parent's
UP counter; acknowledge the children's slots; the root writes the final chunk
into its own result buffer and either into its children's (push) or just bumps
their DOWN counter (pull) — and a *down worker* — wait for DOWN, (pull: copy the
chunk out of the parent's result buffer and acknowledge it with DACK,) hand it
on to the children the same way; a parent whose buffer is pulled from waits for
the last DACK before it returns.  Counters are running totals that are never
reset, so several calls can be simulated back to back on one state.

The workers are Python generators that ``yield`` where the kernel spins on a
flag, and a scheduler interleaves them in a seeded random order, so the model
checks the protocol — no deadlock for any interleaving it tries, no ring slot
refilled before it was read, no chunk read before it is final — as well as the
arithmetic.

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
    ring_depth: int = 4,
    pull_down: bool = False,
    calls: int = 1,
    wait_for_ack: bool = True,
) -> List[np.ndarray]:
    """All-reduce ``inputs`` (one array per rank, same shape) over the double
    binary tree; returns one result array per rank.  ``inputs`` are not
    modified.  ``calls`` > 1 repeats the reduction on the same counters and ring
    (every rank's workers of call ``k + 1`` start when ITS call ``k`` is over, the
    ranks run free of each other), the way back-to-back kernel launches do.
    ``wait_for_ack=False`` drops the flow control of the ring (a child then refills a slot
    whenever it likes): the mistake the ACK counters prevent, for tests of the model itself."""
    W = len(inputs)
    numel = inputs[0].size
    inp = [np.array(x, dtype=acc_dtype, copy=True).reshape(-1) for x in inputs]
    res = [np.zeros(numel, dtype=acc_dtype) for _ in range(W)]
    bounds = chunk_bounds(numel, n_chunks)
    nbr = [[tree_neighbours(W, r, t) for t in (0, 1)] for r in range(W)]
    D = ring_depth

    def chunks_of(tree):
        return [c for c in range(n_chunks) if c % 2 == tree]

    def child_slot(r, t):
        parent = nbr[r][t][0]
        return 0 if parent < 0 or nbr[parent][t][1] == r else 1

    # counters, all written by a *peer* and polled by the owner (as on the GPU); running totals
    up_cnt = [[[0, 0] for _ in range(2)] for _ in range(W)]    # [rank][tree][child slot]
    down_cnt = [[0, 0] for _ in range(W)]                       # [rank][tree]
    ack_cnt = [[0, 0] for _ in range(W)]                        # [rank][tree]: my slots the parent has read
    dack_cnt = [[[0, 0] for _ in range(2)] for _ in range(W)]   # [rank][tree][child slot]: slices a child pulled
    # ring[rank][tree][child slot][g % D] = [running chunk number g, partial, read yet?]
    ring = [[[[None] * D for _ in range(2)] for _ in range(2)] for _ in range(W)]
    final = [[dict() for _ in range(2)] for _ in range(W)]      # chunk -> call whose final value is in res
    progress = [0]

    def up_worker(r, t, call, base):
        parent, left, right = nbr[r][t]
        kids = [(slot, k) for slot, k in enumerate((left, right)) if k >= 0]
        cs = child_slot(r, t)
        for n, c in enumerate(chunks_of(t)):
            g = base + n
            lo, hi = bounds[c]
            for slot, _ in kids:
                while up_cnt[r][t][slot] < g + 1:
                    yield
            if parent >= 0 and wait_for_ack:
                while ack_cnt[r][t] < g + 1 - D:
                    yield
            acc = inp[r][lo:hi].copy()
            for slot, _ in kids:
                entry = ring[r][t][slot][g % D]
                assert entry is not None and entry[0] == g, "ring slot does not hold this chunk's partial"
                acc += entry[1]
                entry[2] = True
            if parent >= 0:
                old = ring[parent][t][cs][g % D]
                assert old is None or old[2], "ring slot refilled before the parent read it"
                ring[parent][t][cs][g % D] = [g, acc, False]
                up_cnt[parent][t][cs] = g + 1
            else:
                res[r][lo:hi] = acc
                final[r][t][c] = call
                for _, k in kids:
                    if not pull_down:
                        res[k][lo:hi] = acc
                        final[k][t][c] = call
                    down_cnt[k][t] = g + 1
            for _, k in kids:
                ack_cnt[k][t] = g + 1
            progress[0] += 1

    def down_worker(r, t, call, base):
        parent, left, right = nbr[r][t]
        kids = [(slot, k) for slot, k in enumerate((left, right)) if k >= 0]
        cs = child_slot(r, t)
        mine = chunks_of(t)
        for n, c in enumerate(mine if parent >= 0 else []):
            g = base + n
            lo, hi = bounds[c]
            while down_cnt[r][t] < g + 1:
                yield
            if pull_down:
                assert final[parent][t].get(c) == call, "pulled a chunk that is not final at the parent"
                res[r][lo:hi] = res[parent][lo:hi]
                final[r][t][c] = call
                dack_cnt[parent][t][cs] = g + 1
            else:
                assert final[r][t].get(c) == call, "DOWN raised before the chunk was stored"
            for _, k in kids:
                if not pull_down:
                    res[k][lo:hi] = res[r][lo:hi]
                    final[k][t][c] = call
                down_cnt[k][t] = g + 1
            progress[0] += 1
        if pull_down and mine:  # nobody may still read this rank's buffer when its kernel returns
            for slot, _ in kids:
                while dack_cnt[r][t][slot] < base + len(mine):
                    yield

    def rank_worker(r):
        """One rank's stream: the workers of call k + 1 start when all of this rank's workers of call k are done."""
        for call in range(calls):
            ws = []
            for t in (0, 1):
                base = call * len(chunks_of(t))
                ws.append(up_worker(r, t, call, base))
                ws.append(down_worker(r, t, call, base))
            while ws:
                rng.shuffle(ws)
                alive = []
                for w_ in ws:
                    try:
                        next(w_)
                        alive.append(w_)
                    except StopIteration:
                        progress[0] += 1
                ws = alive
                if ws:
                    yield

    rng = random.Random(seed)
    ranks = [rank_worker(r) for r in range(W)]
    idle_rounds = 0
    while ranks:
        rng.shuffle(ranks)
        before = progress[0]
        alive = []
        for w_ in ranks:
            try:
                next(w_)
                alive.append(w_)
            except StopIteration:
                progress[0] += 1
        ranks = alive
        idle_rounds = 0 if progress[0] != before else idle_rounds + 1
        if idle_rounds > 8:
            raise _Deadlock("double-tree protocol made no progress")
    return [b.reshape(inputs[0].shape) for b in res]
