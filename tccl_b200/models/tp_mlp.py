"""Tensor-parallel Llama-style MLP block built on the fused kernels.

The reference ships no model; "fuse collectives with matmuls" is the stated
motivation of the project (``presentation.pdf``, slide 4).  This block is that use case, with
Llama-3-8B dimensions as the default (hidden 4096, intermediate 14336):

* sequence-parallel form (``forward``): the input is this rank's token shard
  ``[T / W, hidden]``; **all-gather -> gate/up GEMM + SwiGLU** is one kernel,
  **down GEMM -> reduce-scatter** is one kernel; the output is again a token
  shard.  No stand-alone collective, no elementwise kernel in between.
* all-reduce form (``forward_allreduce``): replicated input, local GEMMs, then
  **all-reduce + bias + residual + RMSNorm** as one kernel.

Weights are random-initialised in the ``nn.Linear`` layout and sliced for the
rank: gate/up are column-parallel (``intermediate / W`` rows each, packed
gate|up per 128 rows for the fused SwiGLU epilogue), down is row-parallel
(``[hidden, intermediate / W]``).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops.fused import all_gather_gemm, all_reduce_bias_residual_rmsnorm, gemm_reduce_scatter, pack_gate_up
from ..ops.gemm import gemm_bf16
from ..parallel.world import WorldBase


class TensorParallelMLP:
    def __init__(self, world: WorldBase, rank: int, hidden: int = 4096, intermediate: int = 14336, seed: int = 4000,
                 device=None, full_weights=None):
        W = world.world_size
        if intermediate % (W * 128):
            raise ValueError("intermediate / world_size must be a multiple of 128")
        self.world, self.rank, self.hidden, self.intermediate = world, rank, hidden, intermediate
        self.inter_local = intermediate // W
        dev = device or world.device
        if full_weights is None:
            full_weights = self.init_full_weights(hidden, intermediate, seed)
        gate, up, down = full_weights
        lo, hi = rank * self.inter_local, (rank + 1) * self.inter_local
        self.gate_w = gate[lo:hi].to(dev)
        self.up_w = up[lo:hi].to(dev)
        self.gate_up_packed = pack_gate_up(self.gate_w, self.up_w)
        self.down_w = down[:, lo:hi].contiguous().to(dev)  # [hidden, inter_local] = bt layout of the down GEMM
        self.norm_w = torch.ones(hidden, dtype=torch.bfloat16, device=dev)

    @staticmethod
    def init_full_weights(hidden: int, intermediate: int, seed: int = 4000):
        """N(0, 0.02) weights of the whole (unsharded) block, generated on the CPU so
        that every rank can slice the same tensors."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        mk = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(torch.bfloat16)
        return mk(intermediate, hidden), mk(intermediate, hidden), mk(hidden, intermediate)

    # -- sequence-parallel in, sequence-parallel out: two fused kernels
    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        act, _ = all_gather_gemm(x_shard, self.gate_up_packed, swiglu=True, world=self.world)
        return gemm_reduce_scatter(act, self.down_w, world=self.world)

    # -- replicated in, replicated out: local GEMMs + one fused all-reduce/norm kernel
    def forward_allreduce(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, eps: float = 1e-5):
        T = x.shape[0]
        gu = gemm_bf16(x, self.gate_up_packed)                     # [T, 2 * inter_local], packed gate|up per 256
        gu = gu.view(T, -1, 2, 128)
        act = (torch.nn.functional.silu(gu[:, :, 0].float()) * gu[:, :, 1].float()).to(torch.bfloat16).reshape(T, -1)
        key = ("partial", T)
        buf = self.__dict__.setdefault("_bufs", {})
        if key not in buf:
            buf[key] = self.world.empty((T, self.hidden), torch.bfloat16)
        gemm_bf16(act, self.down_w, out=buf[key])
        return all_reduce_bias_residual_rmsnorm(buf[key], self.norm_w, None, residual, eps=eps, world=self.world)

    # -- plain PyTorch fp32 reference of the whole (unsharded) block
    @staticmethod
    def reference(x_full: torch.Tensor, full_weights) -> torch.Tensor:
        gate, up, down = (t.float().to(x_full.device) for t in full_weights)
        xf = x_full.float()
        act = torch.nn.functional.silu(xf @ gate.t()) * (xf @ up.t())
        return act @ down.t()
