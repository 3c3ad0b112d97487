"""A one-rank *real* world (process group of size 1 over PyTorch symmetric memory) on one GPU:
exercises the RealWorld code paths — allocation, rendezvous, cached plans, status, reset — and
both forms of the tensor-parallel MLP block against the fp32 reference.  Run as a script by
tests/test_real_world_single.py (its own process, so the process group does not leak)."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import tccl_b200 as tccl  # noqa: E402
from tccl_b200.models import TensorParallelMLP  # noqa: E402


def main():
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(29700 + os.getpid() % 200))
    torch.cuda.set_device(0)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    w = tccl.init()
    assert w.world_size == 1 and tccl.world() is w
    x = tccl.empty(1 << 16, dtype=torch.bfloat16)
    x.normal_()
    keep = x.clone()
    for fn in (lambda: tccl.one_shot_all_reduce(x), lambda: tccl.all_reduce(x), lambda: tccl.double_tree_all_reduce(x),
               lambda: tccl.one_shot_reduce_scatter(x)):
        y = fn()
        assert torch.equal(y, keep), "a one-rank reduction must return its input"
    g = tccl.one_shot_all_gather(x, 1)
    assert g.shape == (1, 1 << 16) and torch.equal(g[0], keep)
    n0 = w.launches
    tccl.all_reduce(x)  # planned above: a cached launch
    assert w.launches == n0 + 1 and len(w.plans) >= 4
    tccl.barrier(blocks=4, rounds=3)
    tccl.barrier_test(w.handle(x), blocks=8)
    torch.cuda.synchronize()
    assert tccl.last_status()["code"] == 0
    w.check()
    tccl.reset()

    hidden, inter, T = 512, 1024, 256
    fw = TensorParallelMLP.init_full_weights(hidden, inter, seed=4000)
    mlp = TensorParallelMLP(w, 0, hidden, inter, full_weights=fw)
    xs = (torch.randn(T, hidden, generator=torch.Generator().manual_seed(5)) * 1.0).to(torch.bfloat16).cuda()
    ref = TensorParallelMLP.reference(xs, fw)
    out = mlp.forward(xs)  # all-gather -> GEMM + SwiGLU, GEMM -> reduce-scatter
    torch.cuda.synchronize()
    err = (out.float() - ref).abs()
    assert bool((err <= ref.abs() * 2 ** -6 + 3e-3).all()), err.max().item()
    resid = (torch.randn(T, hidden, generator=torch.Generator().manual_seed(6))).to(torch.bfloat16).cuda()
    y = mlp.forward_allreduce(xs, residual=resid)  # local GEMMs + all-reduce/residual/RMSNorm kernel
    torch.cuda.synchronize()
    h = ref + resid.float()
    yref = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + 1e-5)
    err = (y.float() - yref).abs()
    assert bool((err <= yref.abs() * 2 ** -5 + 3e-2).all()), err.max().item()
    w.check()
    print("real_world_single: ok, launches", w.launches)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
