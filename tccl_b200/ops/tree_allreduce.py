"""Double-binary-tree all-reduce (pipelined chunks over both trees).

``double_tree_all_reduce(tensor)`` keeps the reference's name and call shape
(``triton_double_tree_allreduce.py:338-370``) but runs the algorithm the
reference only sketches: the neighbours come from
``get_parents_and_children(world_size, rank)`` for the actual world size (the
reference hard-codes 8 and a global ``rank``), and the kernel really reduces up
and broadcasts down both trees.

The reduction happens in place in the symmetric buffer (partials overwrite the
rank's own data on the way up), so by default the input is first copied into a
scratch symmetric buffer and the result is returned as a new tensor, leaving
``tensor`` intact like the reference's wrapper; ``inplace=True`` reduces
``tensor`` itself and skips the copy.
"""
from __future__ import annotations

from typing import Optional

from ..parallel.tree import tree_neighbours
from ..parallel.world import WorldBase
from ..utils import lib as L
from ._common import K, check_sym_tensor, dtype_code, get_world
from .collectives import Plan, _cached, _check_out, _key

__all__ = ["double_tree_all_reduce"]


def _tree_grid(w: WorldBase, nbytes: int):
    """(K, chunk_vecs): CTAs per role and 16-byte vectors per chunk."""
    cfg = w.config
    kmax = min(cfg.tree_ctas, K["TCCL_TREE_MAX_CTAS"], max(1, w.max_ctas() // 4))
    # at least 64 KiB per CTA per chunk, or the per-chunk handshake dominates
    k = max(1, min(kmax, nbytes // (2 * 65536)))
    if cfg.tree_chunk_bytes < 65536:
        chunk_bytes = cfg.tree_chunk_bytes  # small chunks on request (tests of the pipeline)
    else:
        floor = k * 65536
        # keep several chunks per tree in flight even for medium messages
        chunk_bytes = max(floor, min(cfg.tree_chunk_bytes, nbytes // 8))
    chunk_vecs = max(1, chunk_bytes // 16)
    return k, chunk_vecs


def double_tree_all_reduce(tensor, out=None, *, inplace: bool = False, world: Optional[WorldBase] = None):
    w = get_world(world)
    return _cached(w, _key("tree", w, tensor, out, inplace), lambda: _plan(w, tensor, out, inplace))


def _plan(w: WorldBase, x, out, inplace: bool) -> Plan:
    check_sym_tensor(w, x, "double_tree_all_reduce input")
    x0 = w.local(x, w.local_ranks[0])
    dt = dtype_code(x0.dtype)
    nbytes = x0.numel() * x0.element_size()
    if nbytes % 16:
        raise ValueError("the element count must be a whole number of 16-byte vectors")
    W = w.world_size
    work = x
    pre = None
    if not inplace:
        # reduce inside a scratch symmetric buffer so that the caller's tensor survives
        work = w.empty(x0.shape, x0.dtype)

        def pre():
            for r in w.local_ranks:
                w.local(work, r).copy_(w.local(x, r))
    ptrs = w.peer_ptrs(work)
    k, chunk_vecs = _tree_grid(w, nbytes)
    args = {}
    for r in w.local_ranks:
        a = L.TreeArgs()
        for p, v in enumerate(ptrs):
            a.buf[p] = v
        a.numel = x0.numel()
        a.chunk_vecs = chunk_vecs
        a.dtype = dt
        a.ctas_per_role = k
        for t in (0, 1):
            parent, left, right = tree_neighbours(W, r, t)
            a.parent[t], a.left[t], a.right[t] = parent, left, right
            a.child_slot[t] = 0
            if parent >= 0:
                a.child_slot[t] = 0 if tree_neighbours(W, parent, t)[1] == r else 1
        if out is not None:
            o = w.local(out, r)
            _check_out(o, w.local(x, r))
            a.out = o.data_ptr()
        args[r] = a
    go = w.prepare("tccl_allreduce_tree", args, 4 * k, w.config.block, dt)
    result = out if out is not None else work
    if pre is None:
        return Plan(w, go, args, result=result)

    def go2():
        pre()
        go()

    return Plan(w, go2, args, result=result)
