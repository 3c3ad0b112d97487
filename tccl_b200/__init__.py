"""tccl_b200 — Blackwell-native collectives over PyTorch symmetric memory.

Hand-written sm_100a kernels (P2P loads/stores and NVLS ``multimem`` over
NVLink 5 / NVSwitch) behind a ``torch.Tensor``-in / ``torch.Tensor``-out API:
signal-pad barriers, one-shot / two-shot all-reduce, a double-binary-tree
builder and a pipelined double-tree all-reduce, all-gather, reduce-scatter, and
fused compute+collective ops for tensor parallelism.

Typical use (one process per GPU, started by torchrun)::

    dist.init_process_group("nccl")
    import tccl_b200 as tccl
    tccl.init()
    x = tccl.empty(1 << 20, dtype=torch.bfloat16).normal_()
    y = tccl.one_shot_all_reduce(x)
"""
from __future__ import annotations

from typing import Optional

from .config import Config
from .parallel.tree import build_double_tree, build_tree, get_parents_and_children
from .parallel.simulate import simulate_double_tree_all_reduce

__version__ = "0.1.0"


def init(group=None, config: Optional[Config] = None):
    """Create the default communicator for ``group`` (collective call)."""
    from .ops._common import set_default_world
    from .parallel.world import RealWorld

    w = RealWorld(group=group, config=config)
    set_default_world(w)
    return w


def world():
    from .ops._common import get_world

    return get_world()


def empty(shape, dtype=None):
    import torch

    return world().empty(shape, dtype or torch.bfloat16)


def reset():
    world().reset()


def last_status():
    return world().last_status()


def __getattr__(name):
    # op wrappers import torch + the native library; resolve them lazily so that the
    # CPU-only parts (tree builder, simulator) work without either
    import importlib

    ops = importlib.import_module(".ops", __name__)
    if hasattr(ops, name):
        return getattr(ops, name)
    for mod in ("ops.tree_allreduce", "ops.fused", "ops.gemm", "ops.quantized"):
        try:
            m = importlib.import_module("." + mod, __name__)
        except ImportError:
            continue
        if hasattr(m, name):
            return getattr(m, name)
    raise AttributeError(f"module 'tccl_b200' has no attribute {name!r}")
