"""Double-binary-tree all-reduce (pipelined chunks over both trees).

``double_tree_all_reduce(tensor)`` keeps the reference's name and call shape
(``triton_double_tree_allreduce.py:338-370``) but runs the algorithm the
reference only sketches: the neighbours come from
``get_parents_and_children(world_size, rank)`` for the actual world size (the
reference hard-codes 8 and a global ``rank``), and the kernel really reduces up
and broadcasts down both trees.

Data moves by stores into the receiver's memory only: a rank reads nothing but
its own input, partial sums travel through a ring in the communicator's
workspace, and a parent stores the final value into its children's *result
buffer*, which therefore lives in symmetric memory: ``tensor`` itself with
``inplace=True``, else a scratch buffer shared by all calls of one size, from
which the kernel copies each slice into an ordinary output tensor (a fresh one
per call unless ``out=`` is given), so ``tensor`` stays intact like the
reference's wrapper and two results never alias.  Only the in-place form needs
``tensor`` in symmetric memory.  (``tree_pull_min_bytes`` switches the way down
to the other form: children load the sum from the parent's result buffer.)

Messages up to ``tree_ll_max_bytes`` (2 MiB) take a kernel of their own whose
16-byte lines carry the call number next to the data (``tree_allreduce_ll.cu``):
no counters, no fences, and nothing has to be symmetric, in place or not.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..parallel.tree import tree_neighbours
from ..parallel.world import WorldBase
from ..utils import lib as L
from ._common import K, check_sym_tensor, dtype_code, get_world
from .collectives import _OUT, _X, Plan, _cached, _check_out, _key

__all__ = ["double_tree_all_reduce"]

_SLICE = K["TCCL_TREE_SLICE_BYTES"]
_LL_SLOT = K["TCCL_TREE_LL_SLOT_BYTES"]


def _tree_grid(w: WorldBase, nbytes: int):
    """(K, chunk_vecs): CTAs per role and 16-byte vectors per chunk.  A CTA moves at most one
    ring slice (``TCCL_TREE_SLICE_BYTES``, 256 KiB) of a chunk; small messages use few CTAs (latency), large ones all the
    ring serves, with at least four chunks per tree so that the up and down phases overlap."""
    cfg = w.config
    kmax = max(1, min(cfg.tree_ctas, K["TCCL_TREE_MAX_CTAS"], max(1, w.max_ctas() // 4)))
    per_tree = max(16, nbytes // 2)
    if cfg.tree_chunk_bytes < _SLICE:  # small chunks on request (tests of the pipeline)
        chunk_bytes = max(16, cfg.tree_chunk_bytes // 16 * 16)
        k = max(1, min(kmax, chunk_bytes // 16))
        return k, chunk_bytes // 16
    k = max(1, min(kmax, per_tree // 32768))
    slice_bytes = max(4096, min(_SLICE, per_tree // k // 4, cfg.tree_chunk_bytes // k))
    slice_bytes = max(16, slice_bytes // 16 * 16)
    return k, k * slice_bytes // 16


def double_tree_all_reduce(tensor, out=None, *, inplace: bool = False, world: Optional[WorldBase] = None):
    w = get_world(world)
    cfg = w.config  # the settings that shape the plan are part of its key
    knobs = (cfg.tree_ll_max_bytes, cfg.tree_pull_min_bytes, cfg.tree_ctas, cfg.tree_chunk_bytes)
    return _cached(w, _key("tree", w, tensor, out, inplace, knobs), lambda: _plan(w, tensor, out, inplace), tensor, out)


def _plan(w: WorldBase, x, out, inplace: bool) -> Plan:
    x0 = w.local(x, w.local_ranks[0])
    if not x0.is_cuda or not x0.is_contiguous() or x0.data_ptr() % 16:
        raise ValueError("the input must be a contiguous, 16-byte aligned CUDA tensor")
    dt = dtype_code(x0.dtype)
    nbytes = x0.numel() * x0.element_size()
    if nbytes % 16:
        raise ValueError("the element count must be a whole number of 16-byte vectors")
    W = w.world_size
    if nbytes <= min(w.config.tree_ll_max_bytes, 2 * _ll_max_ctas(w) * (_LL_SLOT // 2)):
        return _plan_ll(w, x, out, inplace, x0, dt, nbytes)
    if inplace:
        # parents store the sum into their children's result buffer: it must be peer-mapped
        check_sym_tensor(w, x, "double_tree_all_reduce(inplace=True) input above the small-message limit")
        work = x
    else:
        # the result buffer that parents store into: one scratch per size and dtype; every
        # call copies its result out inside the kernel, so sharing it is safe
        cache = w.__dict__.setdefault("_tree_work", {})
        key = (x0.numel(), x0.dtype)
        work = cache.get(key)
        if work is None:
            work = cache[key] = w.empty(x0.numel(), x0.dtype)
    ptrs = w.peer_ptrs(work)
    k, chunk_vecs = _tree_grid(w, nbytes)
    args = {}
    for r in w.local_ranks:
        a = L.TreeArgs()
        a.inp = w.local(x, r).data_ptr()
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
    pull = K["TCCL_TREE_PULL_DOWN"] if nbytes >= w.config.tree_pull_min_bytes else 0
    go = w.prepare("tccl_allreduce_tree", args, 4 * k, w.config.block, dt | pull)
    if out is not None:
        return Plan(w, go, args, result=_OUT)
    if inplace:
        return Plan(w, go, args, result=_X)
    shape, dtype, dev = tuple(x0.shape), x0.dtype, x0.device
    return Plan(w, go, args, alloc=lambda r: torch.empty(shape, dtype=dtype, device=dev))


def _neighbours(a, W: int, r: int) -> None:
    for t in (0, 1):
        parent, left, right = tree_neighbours(W, r, t)
        a.parent[t], a.left[t], a.right[t] = parent, left, right
        a.child_slot[t] = 0
        if parent >= 0:
            a.child_slot[t] = 0 if tree_neighbours(W, parent, t)[1] == r else 1


def _ll_max_ctas(w: WorldBase) -> int:
    """CTAs per role the small-message kernel may use: its ring's, and (emulated ranks share one GPU)
    what is resident at once."""
    return max(1, min(K["TCCL_TREE_LL_MAX_CTAS"], w.max_ctas() // 4))


def _plan_ll(w: WorldBase, x, out, inplace: bool, x0, dt: int, nbytes: int) -> Plan:
    """Small message: every line on the wire carries its own flag (``tree_allreduce_ll.cu``); the sums
    come back through the ring too, so the result is written locally and nothing needs a scratch."""
    W = w.world_size
    k = max(1, min(_ll_max_ctas(w), -(-nbytes // 16384)))
    while 2 * k * (_LL_SLOT // 2) < nbytes:
        k += 1
    args = {}
    for r in w.local_ranks:
        a = L.TreeArgs()
        xr = w.local(x, r)
        a.inp = xr.data_ptr()
        a.buf[r] = xr.data_ptr() if inplace else 0
        a.numel = x0.numel()
        a.chunk_vecs = 0
        a.dtype = dt
        a.ctas_per_role = k
        _neighbours(a, W, r)
        if out is not None:
            o = w.local(out, r)
            _check_out(o, xr)
            a.out = o.data_ptr()
        args[r] = a
    block = 128 if nbytes <= 8192 else (256 if nbytes <= 65536 else 512)
    go = w.prepare("tccl_allreduce_tree_ll", args, 4 * k, block, dt)
    if out is not None:
        return Plan(w, go, args, result=_OUT)
    if inplace:
        return Plan(w, go, args, result=_X)
    shape, dtype, dev = tuple(x0.shape), x0.dtype, x0.device
    return Plan(w, go, args, alloc=lambda r: torch.empty(shape, dtype=dtype, device=dev))
