"""Stand-alone tcgen05 GEMM (``c = a @ bt.T``), the mainloop the fused
collective kernels are built on.  bf16 operands, fp32 accumulation in tensor
memory, bf16 result.  The reference has no GEMM; ``presentation.pdf`` (slide 4) names
the fusion of a matmul with its collective as the goal this mainloop serves."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from ..utils import lib as L

__all__ = ["gemm_bf16"]


def gemm_bf16(a: torch.Tensor, bt: torch.Tensor, out: Optional[torch.Tensor] = None, *, ctas: int = 0,
              status: Optional[torch.Tensor] = None, variant: str = "pair") -> torch.Tensor:
    """``out[m, n] = sum_k a[m, k] * bt[n, k]`` on the current GPU.

    ``a`` is ``[M, K]`` and ``bt`` is ``[N, K]`` (the layout of ``nn.Linear.weight``),
    both bf16 with a unit inner stride; ``K`` and ``N`` must be multiples of 8.
    ``variant="pair"``: 256 x 256 tiles on pairs of SMs (``tcgen05.mma.cta_group::2``);
    ``"single"``: 128 x 256 tiles, one CTA each."""
    if a.dtype != torch.bfloat16 or bt.dtype != torch.bfloat16:
        raise TypeError("gemm_bf16 takes bfloat16 operands")
    if a.dim() != 2 or bt.dim() != 2 or a.shape[1] != bt.shape[1]:
        raise ValueError("shapes must be a[M, K], bt[N, K]")
    if a.stride(1) != 1 or bt.stride(1) != 1:
        raise ValueError("operands must have a unit inner stride")
    M, K = a.shape
    N = bt.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    g = L.GemmArgs(a.data_ptr(), bt.data_ptr(), out.data_ptr(), status.data_ptr() if status is not None else 0,
                   M, N, K, a.stride(0), bt.stride(0), out.stride(0))
    stream = torch.cuda.current_stream(a.device).cuda_stream
    if variant not in ("pair", "single"):
        raise ValueError("variant must be 'pair' or 'single'")
    name = "tccl_gemm_bf16_pair" if variant == "pair" else "tccl_gemm_bf16"
    L.check(getattr(L.lib(), name)(C.byref(g), int(ctas), C.c_void_p(stream)), name)
    return out
