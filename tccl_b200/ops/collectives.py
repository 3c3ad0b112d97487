"""Flat collectives over symmetric memory: all-reduce (one-shot / two-shot),
all-gather, reduce-scatter, each with a P2P and an NVLS (multimem) kernel.

Reference API kept (``one_shot_all_reduce``, ``one_shot_all_gather``,
``one_shot_reduce_scatter``: ``triton_one_shot_all_reduce_no_128.py:67-96``,
``triton_all_gather.py:66-95``, ``triton_reduce_scatter.py:95-127``) and
widened: bf16 / fp32 / fp16, fp32 accumulation, any element count (ragged
tails), ``out=`` to avoid the per-call allocation, in-place two-shot, and a
size-based choice of kernel.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..parallel.world import WorldBase
from ..utils import lib as L
from ._common import K, check_sym_tensor, dtype_code, get_world, grid_for

__all__ = [
    "all_reduce", "all_gather", "reduce_scatter",
    "one_shot_all_reduce", "one_shot_all_gather", "one_shot_reduce_scatter",
    "choose_all_reduce_algo",
]

_AR_KERNELS = {
    "oneshot_p2p": "tccl_allreduce_oneshot_p2p",
    "oneshot_nvls": "tccl_allreduce_oneshot_nvls",
    "twoshot_p2p": "tccl_allreduce_twoshot_p2p",
    "twoshot_nvls": "tccl_allreduce_twoshot_nvls",
}


def _base_args(world: WorldBase, x, dt: int, flags: int) -> L.CollArgs:
    a = L.CollArgs()
    ptrs = world.peer_ptrs(x)
    for p, v in enumerate(ptrs):
        a.inp[p] = v
    a.mc_in = world.mc_ptr(x)
    a.numel = world.local(x, world.local_ranks[0]).numel()
    a.dtype = dt
    a.flags = flags
    return a


def _copy_args(a: L.CollArgs) -> L.CollArgs:
    b = L.CollArgs()
    import ctypes as C
    C.memmove(C.byref(b), C.byref(a), C.sizeof(a))
    return b


def choose_all_reduce_algo(world: WorldBase, nbytes: int, symmetric_dst: bool) -> str:
    """Size-based choice.  One-shot moves (W-1) S into every GPU but needs one
    barrier round trip less and no symmetric destination: best for small
    messages.  Two-shot moves about 2 (W-1)/W S (P2P) or S (NVLS) and needs a
    symmetric destination (the input itself when in place)."""
    cfg = world.config
    if cfg.force_variant:
        return cfg.force_variant
    nvls = world.has_nvls
    if world.world_size == 1:
        return "oneshot_p2p"
    if not symmetric_dst or nbytes <= cfg.oneshot_max_bytes:
        return "oneshot_nvls" if nvls and nbytes <= 4 * cfg.oneshot_max_bytes else "oneshot_p2p"
    return "twoshot_nvls" if nvls else "twoshot_p2p"


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
    check_sym_tensor(w, x, "all_reduce input")
    x0 = w.local(x, w.local_ranks[0])
    dt = dtype_code(x0.dtype)
    nbytes = x0.numel() * x0.element_size()
    if algo == "tree":
        from .tree_allreduce import double_tree_all_reduce

        return double_tree_all_reduce(x, out=out, inplace=inplace, world=w)
    out_is_sym = out is not None and _is_symmetric(w, out)
    sym_dst = inplace or out_is_sym
    if algo == "auto":
        algo = choose_all_reduce_algo(w, nbytes, sym_dst)
    if algo not in _AR_KERNELS:
        raise ValueError(f"unknown all-reduce algo {algo!r}")
    if algo.endswith("nvls") and not w.has_nvls:
        raise RuntimeError(f"{algo} needs NVLS multicast, which this world does not have")
    flags = w.coll_flags(sync_exit=sync_exit)
    base = _base_args(w, x, dt, flags)
    vpt = 16 // x0.element_size()
    nvec = x0.numel() // vpt
    block = w.config.block
    per_rank = {}
    if algo.startswith("oneshot"):
        if inplace:
            # a one-shot result cannot land in the buffer peers are still reading: stage it
            tmp = {r: torch.empty_like(w.local(x, r)) for r in w.local_ranks}
            res = _launch_oneshot(w, algo, base, tmp, nvec, block, dt)
            for r in w.local_ranks:
                w.local(x, r).copy_(res[r])
            return x
        outs = {}
        for r in w.local_ranks:
            o = w.local(out, r) if out is not None else torch.empty_like(w.local(x, r))
            _check_out(o, w.local(x, r))
            outs[r] = o
        _launch_oneshot(w, algo, base, outs, nvec, block, dt)
        return out if out is not None else w.wrap(outs)
    # two-shot: destination must be symmetric
    if not sym_dst:
        raise ValueError("two-shot all-reduce writes into symmetric memory: pass inplace=True or a symmetric out")
    dst = x if inplace else out
    check_sym_tensor(w, dst, "all_reduce destination")
    dptrs = w.peer_ptrs(dst)
    args = {}
    for r in w.local_ranks:
        a = _copy_args(base)
        for p, v in enumerate(dptrs):
            a.out_peer[p] = v
        a.mc_out = w.mc_ptr(dst)
        args[r] = a
    per_slice = -(-nvec // w.world_size)
    grid = grid_for(w, per_slice, block, 4)
    w.launch(_AR_KERNELS[algo], args, grid, block, dt)
    return dst


def _launch_oneshot(w, algo, base, outs, nvec, block, dt):
    args = {}
    for r, o in outs.items():
        a = _copy_args(base)
        a.out = o.data_ptr()
        args[r] = a
    grid = grid_for(w, nvec, block, 4)
    w.launch(_AR_KERNELS[algo], args, grid, block, dt)
    return outs


def _check_out(o: torch.Tensor, like: torch.Tensor, numel: Optional[int] = None) -> None:
    n = like.numel() if numel is None else numel
    if o.dtype != like.dtype or o.numel() != n or not o.is_contiguous() or o.data_ptr() % 16:
        raise ValueError("out must be contiguous, 16-byte aligned, of the input's dtype and the right size")


def _is_symmetric(w: WorldBase, t) -> bool:
    from ..parallel.emu import EmuTensor

    if isinstance(t, EmuTensor):
        return True
    try:
        w.peer_ptrs(t)
        return True
    except Exception:
        return False


def all_gather(x, out=None, *, algo: str = "auto", world: Optional[WorldBase] = None, sync_exit: bool = True):
    """Gather every rank's ``x`` into a ``(W, *x.shape)`` tensor on every rank.

    ``algo="pull"`` reads the peers' shards into an ordinary local ``out``.
    ``algo="push"`` / ``"push_nvls"`` store the own shard into every rank's
    ``out``, which must then be in symmetric memory.  ``auto``: push when ``out``
    is symmetric and the shard is small (stores are posted, loads are round
    trips), pull otherwise.
    """
    w = get_world(world)
    check_sym_tensor(w, x, "all_gather input")
    x0 = w.local(x, w.local_ranks[0])
    dt = dtype_code(x0.dtype)
    W = w.world_size
    nbytes = x0.numel() * x0.element_size()
    out_is_sym = out is not None and _is_symmetric(w, out)
    if algo == "auto":
        if out_is_sym and nbytes <= (1 << 20):
            algo = "push_nvls" if w.has_nvls else "push"
        else:
            algo = "pull"
    flags = w.coll_flags(sync_exit=sync_exit)
    base = _base_args(w, x, dt, flags)
    vpt = 16 // x0.element_size()
    nvec = x0.numel() // vpt
    block = w.config.block
    if algo == "pull":
        outs, args = {}, {}
        for r in w.local_ranks:
            xr = w.local(x, r)
            o = w.local(out, r) if out is not None else torch.empty((W, *xr.shape), dtype=xr.dtype, device=xr.device)
            _check_out(o, xr, xr.numel() * W)
            a = _copy_args(base)
            a.out = o.data_ptr()
            outs[r], args[r] = o, a
        w.launch("tccl_allgather_pull_p2p", args, grid_for(w, nvec, block, 4), block, dt)
        return out if out is not None else w.wrap(outs)
    if algo not in ("push", "push_nvls"):
        raise ValueError(f"unknown all-gather algo {algo!r}")
    if not out_is_sym:
        raise ValueError("push all-gather stores into the peers' output: out must be in symmetric memory")
    if algo == "push_nvls" and not w.has_nvls:
        raise RuntimeError("push_nvls needs NVLS multicast")
    check_sym_tensor(w, out, "all_gather output")
    if x0.numel() * x0.element_size() % 16:
        raise ValueError("push all-gather needs a shard size that is a multiple of 16 bytes")
    optrs = w.peer_ptrs(out)
    args = {}
    for r in w.local_ranks:
        a = _copy_args(base)
        for p, v in enumerate(optrs):
            a.out_peer[p] = v
        a.mc_out = w.mc_ptr(out)
        args[r] = a
    name = "tccl_allgather_push_nvls" if algo == "push_nvls" else "tccl_allgather_push_p2p"
    w.launch(name, args, grid_for(w, nvec, block, 4), block, dt)
    return out


def reduce_scatter(x, out=None, *, algo: str = "auto", world: Optional[WorldBase] = None, sync_exit: bool = True):
    """Rank r receives ``sum_ranks x[r * n/W : (r+1) * n/W]`` (flattened ``x``).

    As in the reference the element count must be a multiple of ``W`` times the
    16-byte vector width (``triton_reduce_scatter.py:102-104``)."""
    w = get_world(world)
    check_sym_tensor(w, x, "reduce_scatter input")
    x0 = w.local(x, w.local_ranks[0])
    dt = dtype_code(x0.dtype)
    W = w.world_size
    vpt = 16 // x0.element_size()
    if x0.numel() % (vpt * W):
        raise ValueError(f"numel must be a multiple of {vpt * W} (vector width x world size)")
    per = x0.numel() // W
    if algo == "auto":
        algo = w.config.force_variant or ("nvls" if w.has_nvls else "p2p")
    if algo not in ("p2p", "nvls"):
        raise ValueError(f"unknown reduce-scatter algo {algo!r}")
    if algo == "nvls" and not w.has_nvls:
        raise RuntimeError("nvls reduce-scatter needs NVLS multicast")
    flags = w.coll_flags(sync_exit=sync_exit)
    base = _base_args(w, x, dt, flags)
    outs, args = {}, {}
    for r in w.local_ranks:
        xr = w.local(x, r)
        o = w.local(out, r) if out is not None else torch.empty(per, dtype=xr.dtype, device=xr.device)
        _check_out(o, xr, per)
        a = _copy_args(base)
        a.out = o.data_ptr()
        outs[r], args[r] = o, a
    block = w.config.block
    name = "tccl_reducescatter_nvls" if algo == "nvls" else "tccl_reducescatter_p2p"
    w.launch(name, args, grid_for(w, per // vpt, block, 4), block, dt)
    return out if out is not None else w.wrap(outs)


# ---- reference-named entry points -------------------------------------------
def one_shot_all_reduce(tensor, out=None, world: Optional[WorldBase] = None):
    """``out = sum over ranks of tensor``; returns a new ordinary tensor."""
    w = get_world(world)
    algo = w.config.force_variant if w.config.force_variant.startswith("oneshot") else (
        "oneshot_nvls" if w.has_nvls and w.world_size > 1 else "oneshot_p2p")
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
