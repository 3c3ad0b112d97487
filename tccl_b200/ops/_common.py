"""Helpers shared by the op wrappers: validation, grid sizing, default world."""
from __future__ import annotations

from typing import Optional

import torch

from ..parallel.world import WorldBase
from ..utils import lib as L

K = L.K
_default_world: Optional[WorldBase] = None


def set_default_world(w: Optional[WorldBase]) -> None:
    global _default_world
    _default_world = w


def get_world(world: Optional[WorldBase] = None) -> WorldBase:
    w = world if world is not None else _default_world
    if w is None:
        raise RuntimeError("tccl_b200 is not initialised: call tccl_b200.init() (after init_process_group) "
                           "or pass world=")
    return w


def debug_log(world: WorldBase, msg: str) -> None:
    """One line per *planned* launch (plans are cached, so this is not on the hot path) when
    ``TCCL_DEBUG=1``: which kernel, grid and block were chosen for which message."""
    if world.config.debug:
        import sys

        rank = getattr(world, "rank", "emu")
        print(f"[tccl_b200 rank {rank}] {msg}", file=sys.stderr, flush=True)


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return L.DTYPES[dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {dtype}; supported: bfloat16, float32, float16") from None


def check_sym_tensor(world: WorldBase, x, what: str = "tensor") -> None:
    t = world.local(x, world.local_ranks[0])
    if not t.is_cuda:
        raise ValueError(f"{what} must live on the GPU in symmetric memory")
    if not t.is_contiguous():
        raise ValueError(f"{what} must be contiguous")
    for p in world.peer_ptrs(x):
        if p % 16:
            raise ValueError(f"{what} must start on a 16-byte boundary on every rank (view offset {p % 16})")


def grid_for(world: WorldBase, nvec: int, block: int, per_thread: int, cap: Optional[int] = None) -> int:
    """CTAs for a grid-stride kernel moving ``nvec`` 16-byte vectors, identical
    on every rank (it depends only on the size and the shared configuration)."""
    want = -(-max(nvec, 1) // (block * per_thread))
    m = world.max_ctas()
    if world.world_size == 1:
        m = world.local_copy_ctas()
    if cap:
        m = min(m, cap)
    return max(1, min(want, m))
