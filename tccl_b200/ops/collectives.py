"""Flat collectives over symmetric memory: all-reduce (one-shot / two-shot),
all-gather, reduce-scatter, each with a P2P and an NVLS (multimem) kernel.

Reference API kept (``one_shot_all_reduce``, ``one_shot_all_gather``,
``one_shot_reduce_scatter``: ``triton_one_shot_all_reduce_no_128.py:67-96``,
``triton_all_gather.py:66-95``, ``triton_reduce_scatter.py:95-127``) and
widened: bf16 / fp32 / fp16, fp32 accumulation, any element count (ragged
tails), ``out=`` to avoid the per-call allocation, in-place two-shot, and a
size-based choice of kernel.

Every call resolves to a *plan*: the validated, fully bound kernel launch.
Plans are cached per (tensor address, size, dtype, destination, algorithm), so
a repeated call costs one dictionary lookup and one C call — the reference
instead re-runs ``rendezvous`` and re-specialises its kernel per size on every
call.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Optional

import torch

from ..parallel.world import PlanCache, WorldBase  # noqa: F401  (PlanCache re-exported for tests)
from ..utils import lib as L
from ._common import K, check_sym_tensor, debug_log, dtype_code, get_world, grid_for

__all__ = [
    "all_reduce", "all_gather", "reduce_scatter",
    "one_shot_all_reduce", "one_shot_all_gather", "one_shot_reduce_scatter",
    "choose_all_reduce_algo",
]

_AR_KERNELS = {
    "push_p2p": "tccl_allreduce_push_p2p",
    "push_nvls": "tccl_allreduce_push_nvls",
    "oneshot_p2p": "tccl_allreduce_oneshot_p2p",
    "oneshot_nvls": "tccl_allreduce_oneshot_nvls",
    "twoshot_p2p": "tccl_allreduce_twoshot_p2p",
    "twoshot_nvls": "tccl_allreduce_twoshot_nvls",
    "twoshot_pipe_p2p": "tccl_allreduce_twoshot_pipe_p2p",
    "twoshot_pipe_nvls": "tccl_allreduce_twoshot_pipe_nvls",
    "twoshot_bulk_p2p": "tccl_allreduce_twoshot_bulk",
}


def pipe_bits(cfg, world_size: int, nvls: bool) -> int:
    """Shape of the pipelined two-shot kernel as the bits its launcher and kernel read:
    reducer warps (of 16), shared-memory stages, vectors per reducer thread per stage."""
    nr = max(1, min(15, int(cfg.pipe_reducers)))
    ur = int(cfg.pipe_unroll)
    if ur not in (2, 4, 8):
        raise ValueError("pipe_unroll must be 2, 4 or 8")
    if not nvls and world_size * ur > 32:   # W loads per output vector: keep the registers in bounds
        ur = 4 if world_size * 4 <= 32 else 2
    stages = max(2, min(16, int(cfg.pipe_stages)))
    while stages > 2 and stages * nr * 32 * ur * 16 > 200 * 1024:
        stages -= 1
    return ((nr << K["TCCL_F_PIPE_REDUCERS_SHIFT"]) | ((stages - 1) << K["TCCL_F_PIPE_STAGES_SHIFT"])
            | (ur << K["TCCL_F_PIPE_UNROLL_SHIFT"]))


_X, _OUT = "<the caller's input>", "<the caller's out>"  # Plan.result: hand back an argument of the call


class Plan:
    """A bound launch.  ``run(x, out)`` enqueues it; ``x`` / ``out`` are the tensors of THIS call.

    A plan holds raw addresses, not the caller's ordinary tensors: an activation that was
    all-reduced once must stay free-able, or the caching allocator could never reuse its
    address and every call would plan (and pin) another one.  Tensors in symmetric memory
    may be referenced: the communicator keeps those allocations alive anyway."""

    __slots__ = ("go", "args", "world", "result", "alloc", "post", "custom")

    def __init__(self, world, go, args, result=None, alloc=None, post=None, custom=None):
        self.world, self.go, self.args, self.result, self.alloc, self.post = world, go, args, result, alloc, post
        self.custom = custom  # a complete replacement of run(), for plans that do not fit the pattern

    def run(self, x=None, out=None):
        if self.custom is not None:
            return self.custom(x, out)
        if self.alloc is not None:  # fresh local output(s) per call
            outs = {}
            for r, a in self.args.items():
                o = self.alloc(r)
                a.out = o.data_ptr()
                outs[r] = o
            self.go()
            return self.world.wrap(outs)
        self.go()
        if self.post is not None:
            self.post(x, out)
        res = self.result
        return x if res is _X else (out if res is _OUT else res)


def _tkey(t):
    """Address, extent AND layout: a strided view that shares address, element count and dtype
    with a contiguous tensor must not hit that tensor's plan."""
    return (t.data_ptr(), tuple(t.shape), tuple(t.stride()), t.dtype)


def _key(tag, w, x, out, *rest):
    x0 = w.local(x, w.local_ranks[0])
    o0 = None if out is None else w.local(out, w.local_ranks[0])
    return (tag, _tkey(x0), None if o0 is None else _tkey(o0), *rest)


def _cached(w: WorldBase, key, build: Callable[[], Plan], x=None, out=None):
    plans = w.plans
    if plans is None:
        return build().run(x, out)
    p = plans.lookup(key)
    if p is None:
        p = build()
        plans.insert(key, p)
    return p.run(x, out)


def _base_args(world: WorldBase, x, dt: int, flags: int) -> L.CollArgs:
    a = L.CollArgs()
    for p, v in enumerate(world.peer_ptrs(x)):
        a.inp[p] = v
    a.mc_in = world.mc_ptr(x)
    x0 = world.local(x, world.local_ranks[0])
    a.numel = x0.numel()
    a.dtype = dt
    a.flags = flags
    # extents for the bounds checks of the debug build (`debug_shrink_extent` is its test hook)
    a.in_bytes = max(0, x0.numel() * x0.element_size() - world.config.debug_shrink_extent)
    a.out_bytes = x0.numel() * x0.element_size()
    return a


def _copy_args(a: L.CollArgs) -> L.CollArgs:
    b = L.CollArgs()
    C.memmove(C.byref(b), C.byref(a), C.sizeof(a))
    return b


def _check_out(o: torch.Tensor, like: torch.Tensor, numel: Optional[int] = None) -> None:
    n = like.numel() if numel is None else numel
    if o.dtype != like.dtype or o.numel() != n or not o.is_contiguous() or o.data_ptr() % 16:
        raise ValueError("out must be contiguous, 16-byte aligned, of the input's dtype and the right size")


def _is_symmetric(w: WorldBase, t) -> bool:
    """Whether ``t`` is known to live in symmetric memory: allocated by ``world.empty`` or
    resolved before (``world.handle(t)`` registers a tensor from ``symm_mem.empty``).  An
    unknown tensor is treated as ordinary memory rather than probed with a rendezvous."""
    from ..parallel.emu import EmuTensor

    if isinstance(t, EmuTensor):
        return True
    handles = getattr(w, "_handles", None)
    return handles is not None and t.untyped_storage().data_ptr() in handles


def choose_all_reduce_algo(world: WorldBase, nbytes: int, symmetric_dst: bool) -> str:
    """Size-based choice.  One-shot moves (W-1) S into every GPU but needs no
    symmetric destination and touches each byte once: best for small messages.
    Two-shot moves about 2 (W-1)/W S (P2P) or (1 + 1/W) S (NVLS) and needs a
    symmetric destination (the input itself when in place)."""
    cfg = world.config
    if cfg.force_variant:
        return cfg.force_variant
    nvls = world.has_nvls
    if world.world_size == 1:
        return "oneshot_p2p"
    use_nvls = nvls and world.world_size > 2
    if use_nvls and symmetric_dst and nbytes > cfg.nvls_twoshot_min_bytes:
        # measured on 8 x B200: 18.8 us flat from 32 KiB to 512 KiB, against 19-21 us (push) and 21-31 us (one-shot)
        if cfg.pipe_min_bytes and nbytes >= cfg.pipe_min_bytes:
            return "twoshot_pipe_nvls"
        return "twoshot_nvls"
    if nbytes <= cfg.push_max_bytes and nbytes % 16 == 0 and nbytes <= world.push_max_bytes():
        return "push_nvls" if use_nvls else "push_p2p"
    if not symmetric_dst or nbytes <= cfg.oneshot_max_bytes:
        return "oneshot_nvls" if nvls and world.world_size > 2 and nbytes <= 4 * cfg.oneshot_max_bytes else "oneshot_p2p"
    if cfg.pipe_min_bytes and nbytes >= cfg.pipe_min_bytes:
        return "twoshot_pipe_nvls" if use_nvls else "twoshot_pipe_p2p"
    if not use_nvls and world.world_size == 2 and cfg.bulk_min_bytes and nbytes >= cfg.bulk_min_bytes:
        # measured on 2 x B200: bulk copies 807 us against 824 us for thread-issued accesses at 512 MiB
        # (665 vs 651 GB/s), level at 32 MiB, behind below 16 MiB
        return "twoshot_bulk_p2p"
    return "twoshot_nvls" if use_nvls else "twoshot_p2p"


def all_reduce(x, out=None, *, inplace: bool = False, algo: str = "auto", world: Optional[WorldBase] = None,
               sync_exit: bool = True):
    """Sum ``x`` over all ranks.

    ``x`` lives in symmetric memory.  Result placement:

    * ``inplace=True`` — the sum replaces ``x`` on every rank (two-shot or tree).
    * ``out`` in symmetric memory — written by the two-shot kernels; ``x`` is kept.
    * ``out`` an ordinary tensor or ``None`` — one-shot kernels; ``x`` is kept.

    ``sync_exit=False`` drops the trailing barrier: the caller then promises not
    to overwrite ``x`` before every rank has finished the call.
    """
    w = get_world(world)
    if algo == "tree":
        from .tree_allreduce import double_tree_all_reduce

        return double_tree_all_reduce(x, out=out, inplace=inplace, world=w)
    return _cached(w, _key("ar", w, x, out, inplace, algo, sync_exit),
                   lambda: _plan_all_reduce(w, x, out, inplace, algo, sync_exit), x, out)


def _plan_push(w, x, out, inplace, algo) -> Plan:
    """Small-message push all-reduce: the input may be any device tensor."""
    locs = {r: (x if w.plans is not None else x[r]) for r in w.local_ranks}
    x0 = locs[w.local_ranks[0]]
    dt = dtype_code(x0.dtype)
    nbytes = x0.numel() * x0.element_size()
    W = w.world_size
    if not x0.is_contiguous() or x0.data_ptr() % 16 or nbytes % 16:
        raise ValueError("push all-reduce needs a contiguous, 16-byte aligned input of a multiple of 16 bytes")
    if nbytes > w.push_max_bytes():
        raise ValueError(f"push all-reduce handles at most {w.push_max_bytes()} bytes per rank")
    if algo == "push_nvls" and not w.has_nvls:
        raise RuntimeError("push_nvls needs NVLS multicast")
    args = {}
    for r in w.local_ranks:
        a = L.CollArgs()
        a.inp[r] = locs[r].data_ptr()  # the slots are found through the communicator itself
        a.in_bytes = max(0, nbytes - w.config.debug_shrink_extent)
        a.out_bytes = nbytes
        a.numel, a.dtype, a.flags = x0.numel(), dt, w.coll_flags()
        args[r] = a
    nvec = nbytes // 16
    block = 256 if nvec <= 2048 else 512
    grid = grid_for(w, nvec, block, 2, cap=32)
    debug_log(w, f"all_reduce {nbytes} B -> {algo}, grid {grid} x {block}")
    go = w.prepare(_AR_KERNELS[algo], args, grid, block, dt)
    if inplace:
        for r, a in args.items():
            a.out = locs[r].data_ptr()  # each vector is read (into the slots) before the barrier, written after
        return Plan(w, go, args, result=_X)
    if out is not None:
        for r, a in args.items():
            o = w.local(out, r)
            _check_out(o, locs[r])
            a.out = o.data_ptr()
        return Plan(w, go, args, result=_OUT)
    shape, dtype, dev = tuple(x0.shape), x0.dtype, x0.device  # no reference to the caller's tensor
    return Plan(w, go, args, alloc=lambda r: torch.empty(shape, dtype=dtype, device=dev))


def _plan_all_reduce(w, x, out, inplace, algo, sync_exit) -> Plan:
    if algo.startswith("push"):
        return _plan_push(w, x, out, inplace, algo)
    if algo == "auto":
        x00 = x if w.plans is not None else x[w.local_ranks[0]]
        nb0 = x00.numel() * x00.element_size()
        x_sym = _is_symmetric(w, x)
        cand = choose_all_reduce_algo(w, nb0, x_sym and (inplace or (out is not None and _is_symmetric(w, out))))
        if cand.startswith("push") and x00.is_contiguous() and x00.data_ptr() % 16 == 0:
            return _plan_push(w, x, out, inplace, cand)
    check_sym_tensor(w, x, "all_reduce input")
    x0 = w.local(x, w.local_ranks[0])
    dt = dtype_code(x0.dtype)
    nbytes = x0.numel() * x0.element_size()
    out_is_sym = out is not None and _is_symmetric(w, out)
    sym_dst = inplace or out_is_sym
    if algo == "auto":
        if (not sym_dst and w.world_size > 1 and w.config.staged_twoshot and nbytes > w.config.oneshot_max_bytes
                and nbytes <= w.config.staged_max_bytes):
            return _plan_staged_twoshot(w, x, out, sync_exit)
        algo = choose_all_reduce_algo(w, nbytes, sym_dst)
        if algo.startswith("push"):  # not eligible after all (alignment): fall back to the pull one-shot
            algo = "oneshot_nvls" if w.has_nvls and w.world_size > 2 else "oneshot_p2p"
        if algo == "twoshot_bulk_p2p":  # bulk copies start on 16-byte boundaries
            dst0 = x0 if inplace else w.local(out, w.local_ranks[0])
            if x0.data_ptr() % 16 or dst0.data_ptr() % 16:
                algo = "twoshot_p2p"
    if algo not in _AR_KERNELS:
        raise ValueError(f"unknown all-reduce algo {algo!r}")
    if algo.endswith("nvls") and not w.has_nvls:
        raise RuntimeError(f"{algo} needs NVLS multicast, which this world does not have")
    flags = w.coll_flags(sync_exit=sync_exit)
    base = _base_args(w, x, dt, flags)
    vpt = 16 // x0.element_size()
    nvec = x0.numel() // vpt
    block = w.config.block
    if algo.startswith("oneshot"):
        args = {r: _copy_args(base) for r in w.local_ranks}
        grid = grid_for(w, nvec, block, 4)
        debug_log(w, f"all_reduce {nbytes} B -> {algo}, grid {grid} x {block}")
        go = w.prepare(_AR_KERNELS[algo], args, grid, block, dt)
        if inplace:
            # a one-shot result cannot land in the buffer peers are still reading: stage it
            tmp = {r: torch.empty_like(w.local(x, r)) for r in w.local_ranks}
            for r, a in args.items():
                a.out = tmp[r].data_ptr()

            def post(x_, _out):
                for r in w.local_ranks:
                    w.local(x_, r).copy_(tmp[r])

            return Plan(w, go, args, result=_X, post=post)
        if out is not None:
            for r, a in args.items():
                o = w.local(out, r)
                _check_out(o, w.local(x, r))
                a.out = o.data_ptr()
            return Plan(w, go, args, result=_OUT)
        shape, dtype, dev = tuple(x0.shape), x0.dtype, x0.device
        return Plan(w, go, args, alloc=lambda r: torch.empty(shape, dtype=dtype, device=dev))
    # two-shot: destination must be symmetric
    if not sym_dst:
        raise ValueError("two-shot all-reduce writes into symmetric memory: pass inplace=True or a symmetric out")
    dst = x if inplace else out
    check_sym_tensor(w, dst, "all_reduce destination")
    if w.local(dst, w.local_ranks[0]).numel() != x0.numel() or w.local(dst, w.local_ranks[0]).dtype != x0.dtype:
        raise ValueError("all_reduce destination must match the input's size and dtype")
    dptrs = w.peer_ptrs(dst)
    args = {}
    for r in w.local_ranks:
        a = _copy_args(base)
        for p, v in enumerate(dptrs):
            a.out_peer[p] = v
        a.mc_out = w.mc_ptr(dst)
        args[r] = a
    per_slice = -(-nvec // w.world_size)
    if algo.startswith("twoshot_pipe"):
        bits = pipe_bits(w.config, w.world_size, algo.endswith("nvls"))
        for a in args.values():
            a.flags |= bits
        block = 512
        nr = (bits >> K["TCCL_F_PIPE_REDUCERS_SHIFT"]) & 15
        ur = (bits >> K["TCCL_F_PIPE_UNROLL_SHIFT"]) & 15
        cap = w.config.max_ctas or w.config.pipe_ctas
        grid = grid_for(w, per_slice, nr * 32, ur, cap=cap)
        debug_log(w, f"all_reduce {nbytes} B -> {algo}, grid {grid} x {block}, pipe bits {bits:#x}")
        return Plan(w, w.prepare(_AR_KERNELS[algo], args, grid, block, dt | bits), args,
                    result=_X if inplace else _OUT)
    if algo == "twoshot_bulk_p2p":
        lib = L.lib()
        lib.tccl_allreduce_bulk_chunk_bytes.restype = C.c_uint32
        chunk_vecs = int(lib.tccl_allreduce_bulk_chunk_bytes(w.world_size)) // 16
        # ~200 KB of shared memory per CTA: one CTA per SM (emulated ranks share the GPU's SMs)
        cap = w.num_sms() if w.plans is not None else max(1, w.num_sms() // w.world_size)
        grid = grid_for(w, per_slice, chunk_vecs, 1, cap=min(cap, w.config.max_ctas or cap))
        debug_log(w, f"all_reduce {nbytes} B -> {algo}, grid {grid} x 256")
        return Plan(w, w.prepare(_AR_KERNELS[algo], args, grid, 256, dt), args, result=_X if inplace else _OUT)
    if algo == "twoshot_nvls":
        cap = w.config.nvls_ctas if not w.config.max_ctas else None
        grid = grid_for(w, per_slice, block, 8, cap=cap)
    else:
        grid = grid_for(w, per_slice, block, 2 if w.world_size >= 8 else 4)
    debug_log(w, f"all_reduce {nbytes} B -> {algo}, grid {grid} x {block}")
    return Plan(w, w.prepare(_AR_KERNELS[algo], args, grid, block, dt), args, result=_X if inplace else _OUT)


def _plan_staged_twoshot(w, x, out, sync_exit) -> Plan:
    """Large message, ordinary destination: a one-shot kernel would pull (W-1) S into every
    GPU.  Reduce with the two-shot kernel into a cached symmetric buffer instead and copy the
    result out locally (one extra pass over HBM, far cheaper than W/2 times the link traffic)."""
    x0 = w.local(x, w.local_ranks[0])
    cache = w.__dict__.setdefault("_staged_ar", {})
    key = (x0.numel(), x0.dtype)
    buf = cache.get(key)
    if buf is None:
        buf = cache[key] = w.empty(x0.numel(), x0.dtype)
    inner = _plan_all_reduce(w, x, buf, False, choose_all_reduce_algo(w, x0.numel() * x0.element_size(), True), sync_exit)
    if out is not None:
        for r in w.local_ranks:
            _check_out(w.local(out, r), w.local(x, r))

        def post(_x, out_):
            for r in w.local_ranks:
                w.local(out_, r).view(-1).copy_(w.local(buf, r))

        return Plan(w, inner.go, inner.args, result=_OUT, post=post)

    shape, dtype, dev = tuple(x0.shape), x0.dtype, x0.device

    def run_fresh(_x, _out):  # a new output tensor per call, filled from the symmetric buffer
        inner.go()
        outs = {r: torch.empty(shape, dtype=dtype, device=dev) for r in w.local_ranks}
        for r, o in outs.items():
            o.view(-1).copy_(w.local(buf, r))
        return w.wrap(outs)

    return Plan(w, inner.go, inner.args, custom=run_fresh)


def all_gather(x, out=None, *, algo: str = "auto", world: Optional[WorldBase] = None, sync_exit: bool = True):
    """Gather every rank's ``x`` into a ``(W, *x.shape)`` tensor on every rank.

    ``algo="pull"`` reads the peers' shards into an ordinary local ``out``.
    ``algo="push"`` / ``"push_nvls"`` store the own shard into every rank's
    ``out``, which must then be in symmetric memory.  ``auto``: push when ``out``
    is symmetric and the shard is small (stores are posted, loads are round
    trips), pull otherwise.
    """
    w = get_world(world)
    return _cached(w, _key("ag", w, x, out, algo, sync_exit), lambda: _plan_all_gather(w, x, out, algo, sync_exit), x, out)


def _plan_all_gather(w, x, out, algo, sync_exit) -> Plan:
    check_sym_tensor(w, x, "all_gather input")
    x0 = w.local(x, w.local_ranks[0])
    dt = dtype_code(x0.dtype)
    W = w.world_size
    nbytes = x0.numel() * x0.element_size()
    out_is_sym = out is not None and _is_symmetric(w, out)
    if algo == "auto":
        if out_is_sym and nbytes <= (1 << 20) and nbytes % 16 == 0:
            algo = "push_nvls" if w.has_nvls else "push"
        else:
            algo = "pull"
    flags = w.coll_flags(sync_exit=sync_exit)
    base = _base_args(w, x, dt, flags)
    base.out_bytes = nbytes * W
    vpt = 16 // x0.element_size()
    nvec = x0.numel() // vpt
    block = w.config.block
    if algo == "pull":
        args = {r: _copy_args(base) for r in w.local_ranks}
        go = w.prepare("tccl_allgather_pull_p2p", args, grid_for(w, nvec, block, 4), block, dt)
        if out is not None:
            for r, a in args.items():
                o = w.local(out, r)
                _check_out(o, w.local(x, r), x0.numel() * W)
                a.out = o.data_ptr()
            return Plan(w, go, args, result=_OUT)
        shape = (W, *x0.shape)
        return Plan(w, go, args, alloc=lambda r: torch.empty(shape, dtype=x0.dtype, device=x0.device))
    if algo not in ("push", "push_nvls"):
        raise ValueError(f"unknown all-gather algo {algo!r}")
    if not out_is_sym:
        raise ValueError("push all-gather stores into the peers' output: out must be in symmetric memory")
    if algo == "push_nvls" and not w.has_nvls:
        raise RuntimeError("push_nvls needs NVLS multicast")
    check_sym_tensor(w, out, "all_gather output")
    if nbytes % 16:
        raise ValueError("push all-gather needs a shard size that is a multiple of 16 bytes")
    if w.local(out, w.local_ranks[0]).numel() != x0.numel() * W:
        raise ValueError("all_gather output must hold world_size shards")
    optrs = w.peer_ptrs(out)
    args = {}
    for r in w.local_ranks:
        a = _copy_args(base)
        for p, v in enumerate(optrs):
            a.out_peer[p] = v
        a.mc_out = w.mc_ptr(out)
        args[r] = a
    name = "tccl_allgather_push_nvls" if algo == "push_nvls" else "tccl_allgather_push_p2p"
    return Plan(w, w.prepare(name, args, grid_for(w, nvec, block, 4), block, dt), args, result=_OUT)


def reduce_scatter(x, out=None, *, algo: str = "auto", world: Optional[WorldBase] = None, sync_exit: bool = True):
    """Rank r receives ``sum_ranks x[r * n/W : (r+1) * n/W]`` (flattened ``x``).

    As in the reference the element count must be a multiple of ``W`` times the
    16-byte vector width (``triton_reduce_scatter.py:102-104``)."""
    w = get_world(world)
    return _cached(w, _key("rs", w, x, out, algo, sync_exit), lambda: _plan_reduce_scatter(w, x, out, algo, sync_exit),
                   x, out)


def _plan_reduce_scatter(w, x, out, algo, sync_exit) -> Plan:
    check_sym_tensor(w, x, "reduce_scatter input")
    x0 = w.local(x, w.local_ranks[0])
    dt = dtype_code(x0.dtype)
    W = w.world_size
    vpt = 16 // x0.element_size()
    if x0.numel() % (vpt * W):
        raise ValueError(f"numel must be a multiple of {vpt * W} (vector width x world size)")
    per = x0.numel() // W
    if algo == "auto":
        algo = w.config.force_variant or ("nvls" if w.has_nvls and W > 2 else "p2p")
    if algo not in ("p2p", "nvls"):
        raise ValueError(f"unknown reduce-scatter algo {algo!r}")
    if algo == "nvls" and not w.has_nvls:
        raise RuntimeError("nvls reduce-scatter needs NVLS multicast")
    flags = w.coll_flags(sync_exit=sync_exit)
    base = _base_args(w, x, dt, flags)
    base.out_bytes = per * x0.element_size()
    args = {r: _copy_args(base) for r in w.local_ranks}
    block = w.config.block
    name = "tccl_reducescatter_nvls" if algo == "nvls" else "tccl_reducescatter_p2p"
    go = w.prepare(name, args, grid_for(w, per // vpt, block, 4), block, dt)
    if out is not None:
        for r, a in args.items():
            o = w.local(out, r)
            _check_out(o, w.local(x, r), per)
            a.out = o.data_ptr()
        return Plan(w, go, args, result=_OUT)
    return Plan(w, go, args, alloc=lambda r: torch.empty(per, dtype=x0.dtype, device=x0.device))


# ---- reference-named entry points -------------------------------------------
def one_shot_all_reduce(tensor, out=None, world: Optional[WorldBase] = None):
    """``out = sum over ranks of tensor``; returns a new ordinary tensor."""
    w = get_world(world)
    algo = w.config.force_variant if w.config.force_variant.startswith("oneshot") else (
        "oneshot_nvls" if w.has_nvls and w.world_size > 2 else "oneshot_p2p")
    return all_reduce(tensor, out=out, algo=algo, world=w)


def one_shot_all_gather(tensor, world_size: Optional[int] = None, out=None, world: Optional[WorldBase] = None):
    """Returns ``(world_size, *tensor.shape)``.  ``world_size`` is accepted for
    signature parity with the reference and must match the communicator."""
    w = get_world(world)
    if world_size is not None and world_size != w.world_size:
        raise ValueError(f"world_size={world_size} does not match the communicator ({w.world_size})")
    return all_gather(tensor, out=out, algo="pull", world=w)


def one_shot_reduce_scatter(tensor, out=None, world: Optional[WorldBase] = None):
    return reduce_scatter(tensor, out=out, world=world)
