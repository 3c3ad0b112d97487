"""Error bounds that follow from the arithmetic of the kernels, shared by the tests and the
benchmarks (a result is checked before it is timed)."""
from __future__ import annotations

import torch

__all__ = ["allreduce_rmsnorm_check"]


def allreduce_rmsnorm_check(y, h_out, partials_sum, bias, residual, weight, eps: float, world: int, nvls: bool):
    """Check ``y, h_out = all_reduce_bias_residual_rmsnorm(..., residual_out=True)`` element-wise.

    ``partials_sum``: the fp32 sum of every rank's partial (``s``).  With ``h = s + bias + residual``:

    * P2P kernels sum the whole of ``h`` in fp32 and round to nearest once: ``|h_out - h| <= 2^-8 |h|``.
    * NVLS kernels get ``s`` back from the switch already in bf16, within one ulp of ``s`` (its
      conversion is not round-to-nearest), add bias and residual in fp32 and round to nearest:
      ``|h_out - h| <= 2^-7 |s| + 2^-8 (|h| + 2^-7 |s|)``.  Where the partials cancel, ``|s|`` is far
      larger than ``|h|``, so a bound relative to the result alone cannot hold.
    * ``y`` is the RMSNorm of the ``h_out`` the kernel kept, rounded once: ``2^-7 |y|`` covers that
      rounding and the fp32 mean.

    Returns ``(ok, worst)`` with ``worst`` the largest error / bound ratio of the pre-norm sum."""
    s = partials_sum.float()
    h = s
    if bias is not None:
        h = h + bias.float()
    if residual is not None:
        h = h + residual.float()
    if nvls:
        bound = 2 ** -7 * s.abs() + 2 ** -8 * (h.abs() + 2 ** -7 * s.abs()) + 1e-6 * world
    else:
        bound = 2 ** -8 * h.abs() + 1e-6 * world
    err = (h_out.float() - h).abs()
    worst = float((err / bound).max())
    ok = bool((err <= bound).all())
    hb = h_out.float()
    ref = hb * torch.rsqrt((hb * hb).mean(-1, keepdim=True) + eps) * weight.float()
    ok = ok and bool(((y.float() - ref).abs() <= ref.abs() * 2 ** -7 + 1e-3).all())
    return ok, worst
