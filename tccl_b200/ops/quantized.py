"""All-reduce with a quantised wire format (fp8 e4m3 + one fp32 scale per 2048
elements on NVLink, fp32 accumulation, bf16 in and out).

"Quantized communication" is named by the reference as a reason for writing
collectives as kernels (``presentation.pdf``, slide 4) but not built there.
``quantized_all_reduce`` trades precision for link bytes: per GPU and direction
``2 (W-1)/W`` bytes per element cross NVLink instead of ``2 (1 + 1/W)`` (bf16
NVLS two-shot) or ``4 (W-1)/W`` (bf16 P2P two-shot).  Every value is rounded to
e4m3 twice (once as a partial, once as the sum), each time with an error of at
most 2^-4 of its chunk's absolute maximum; every rank receives the same bits.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from ..parallel.world import WorldBase
from ..utils import lib as L
from ._common import get_world
from .fused import _locals, _stage_handoff

__all__ = ["quantized_all_reduce", "QUANT_CHUNK"]

QUANT_CHUNK = 2048  # elements per scale


class QarArgs(C.Structure):
    _fields_ = [("inp", C.c_uint64), ("out", C.c_uint64), ("numel", C.c_uint64), ("flags", C.c_int32)]


def quantized_all_reduce(x, out=None, *, world: Optional[WorldBase] = None):
    """Sum ``x`` (bf16, any device memory, ``numel % 2048 == 0``) over all ranks with fp8 on the
    wire; returns a bf16 tensor (``out`` or a new one).  ``out`` may be ``x`` itself."""
    w = get_world(world)
    W = w.world_size
    xs = _locals(w, x)
    x0 = xs[w.local_ranks[0]]
    if x0.dtype != torch.bfloat16:
        raise TypeError("quantized_all_reduce takes bfloat16 tensors")
    n = x0.numel()
    if n == 0 or n % QUANT_CHUNK or not x0.is_contiguous() or x0.data_ptr() % 16:
        raise ValueError(f"the input must be contiguous, 16-byte aligned, with numel % {QUANT_CHUNK} == 0")
    lib = L.lib()
    lib.tccl_allreduce_fp8wire_stage_bytes.restype = C.c_uint64
    need = lib.tccl_allreduce_fp8wire_stage_bytes(C.c_uint64(n), W)
    have = (w.config.stage_mb << 20) - w.ll_bytes
    if need > have:
        raise ValueError(f"staging area too small: need {need >> 20} MiB, have {have >> 20} MiB (raise TCCL_STAGE_MB)")
    outs = {}
    os_ = _locals(w, out) if out is not None else None
    args = {}
    for r in w.local_ranks:
        o = os_[r] if os_ is not None else torch.empty_like(xs[r])
        if o.dtype != torch.bfloat16 or o.numel() != n or not o.is_contiguous() or o.data_ptr() % 16:
            raise ValueError("out must be a contiguous, 16-byte aligned bf16 tensor of the input's size")
        outs[r] = o
        args[r] = QarArgs(xs[r].data_ptr(), o.data_ptr(), n, 0)
    _stage_handoff(w, "fp8wire")
    cps = -(-(n // QUANT_CHUNK) // W)
    grid = max(1, min(-(-cps // 8), 2 * w.max_ctas()))  # a CTA's 8 warps take 8 chunks at a time
    w.launch("tccl_allreduce_fp8wire", args, grid, 256)
    if out is not None:
        return out
    return w.wrap(outs)
