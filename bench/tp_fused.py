"""Tensor-parallel fused paths with Llama-3-8B MLP shapes (bf16, 4096 tokens):

  (a) down-proj GEMM [4096 x I/W] . [I/W x 4096] -> reduce-scatter along tokens
  (b) all-gather of [4096/W x 4096] shards -> up-proj GEMM [4096 x 4096] . [4096 x I/W]
  (c) all-reduce of [4096 x 4096] + bias + residual + RMSNorm (eps 1e-5)

each as ONE fused kernel of this library against the unfused library sequence
(cuBLAS GEMM + NCCL collective [+ torch elementwise/norm kernels]) on the same
GPUs.  Activations N(0,1), weights N(0,0.02), seed 4000 + rank.  Timing: CUDA
events per iteration, p50 of the per-iteration maximum over ranks.  Roofline =
the slower of FLOPs / measured GEMM peak and NVLink bytes / link bandwidth.

    python -m torch.distributed.run --nproc-per-node 8 bench/tp_fused.py --out results/tp8.jsonl
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import tccl_b200 as tccl  # noqa: E402
from tccl_b200.utils.timing import L2Flusher, max_over_ranks, summarize, time_iters  # noqa: E402


def rnd(shape, seed, scale=1.0, device="cuda"):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).to(device)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--intermediate", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--gemm-tflops", type=float, default=1391.6, help="measured sustained cuBLAS bf16 peak")
    ap.add_argument("--link-gbs", type=float, default=770.0)
    ap.add_argument("--flush-l2", type=int, default=1)
    ap.add_argument("--ag-comm-ctas", default="0", help="comma list of data-mover CTA counts to try for (b); 0 = auto")
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    W = int(os.environ.get("WORLD_SIZE", 1))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29544")
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", rank=rank, world_size=W, device_id=torch.device("cuda", local_rank))
    w = tccl.init()
    T, H, I = a.tokens, a.hidden, a.intermediate
    Il = I // W
    rows = T // W
    flush = L2Flusher("cuda") if a.flush_l2 else None
    sync = dist.barrier
    rows_out = []

    def emit(r):
        rows_out.append(r)
        if rank == 0:
            print(json.dumps(r), flush=True)

    def timeit(fn):
        return summarize(max_over_ranks(time_iters(fn, a.iters, a.warmup, before=flush, sync=sync)))

    def report(name, impl, st, flops, link_bytes, ok):
        t = st["p50_us"] * 1e-6
        t_c = flops / (a.gemm_tflops * 1e12) if flops else 0.0
        t_l = link_bytes / (a.link_gbs * 1e9) if W > 1 else 0.0
        roof = max(t_c, t_l)
        emit({"op": name, "impl": impl, "world": W, "p50_us": round(st["p50_us"], 2), "p10_us": round(st["p10_us"], 2),
              "p90_us": round(st["p90_us"], 2), "tflops": round(flops / t / 1e12, 1) if flops else None,
              "roofline_us": round(roof * 1e6, 2), "roofline_frac": round(roof / t, 3) if roof else None,
              "bound": "compute" if t_c >= t_l else "nvlink", "verified": ok})

    # ---------------- (a) GEMM -> reduce-scatter
    acts = [rnd((T, Il), 4000 + r) for r in range(W)] if T * Il * W <= (1 << 28) else None
    a_r = rnd((T, Il), 4000 + rank)
    wd_r = rnd((H, Il), 5000 + rank, 0.02)
    out = tccl.gemm_reduce_scatter(a_r, wd_r, variant="single")
    torch.cuda.synchronize()
    ref = torch.zeros(rows, H, dtype=torch.float32, device="cuda")
    for r in range(W):
        ar = rnd((T, Il), 4000 + r)[rank * rows:(rank + 1) * rows].float()
        ref += ar @ rnd((H, Il), 5000 + r, 0.02).float().t()
    err = (out.float() - ref).abs()
    ok_a = bool((err <= ref.abs() * 2 ** -7 + 0.02 * W).all())
    del ref, acts
    flops = 2.0 * T * H * Il
    link = (W - 1) / W * T * H * 2
    o_buf = torch.empty(rows, H, dtype=torch.bfloat16, device="cuda")
    for variant in ("pair", "single"):
        if variant == "pair" and T % (256 * W):
            continue
        chk = tccl.gemm_reduce_scatter(a_r, wd_r, variant=variant)
        torch.cuda.synchronize()
        ok_v = ok_a and bool(torch.equal(chk, out) or ((chk.float() - out.float()).abs() <= out.float().abs() * 2 ** -7 + 1e-2).all())
        report("gemm_reduce_scatter", f"tccl_b200 fused ({variant})",
               timeit(lambda: tccl.gemm_reduce_scatter(a_r, wd_r, out=o_buf, variant=variant)), flops, link, ok_v)
    part = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")

    def unfused_a():
        torch.matmul(a_r, wd_r.t(), out=part)
        dist.reduce_scatter_tensor(o_buf, part)
    report("gemm_reduce_scatter", "cublas + nccl", timeit(unfused_a), flops, link, True)
    report("gemm_only", "cublas", timeit(lambda: torch.matmul(a_r, wd_r.t(), out=part)), flops, 0, True)
    report("gemm_only", "tccl_b200 tcgen05 (pair)", timeit(lambda: tccl.gemm_bf16(a_r, wd_r, out=part)), flops, 0, True)
    report("gemm_only", "tccl_b200 tcgen05 (single)",
           timeit(lambda: tccl.gemm_bf16(a_r, wd_r, out=part, variant="single")), flops, 0, True)

    # ---------------- (b) all-gather -> GEMM
    x_sh = rnd((rows, H), 4000 + rank)
    wu_r = rnd((Il, H), 6000 + rank, 0.02)
    res, a_full = tccl.all_gather_gemm(x_sh, wu_r, variant="single")
    torch.cuda.synchronize()
    x_all = torch.cat([rnd((rows, H), 4000 + r) for r in range(W)])
    ref = x_all.float() @ wu_r.float().t()
    err = (res.float() - ref).abs()
    ok_b = bool((err <= ref.abs() * 2 ** -8 + 1e-2).all()) and bool(torch.equal(a_full, x_all))
    del ref
    flops = 2.0 * T * H * Il
    link = (W - 1) * rows * H * 2
    o2 = torch.empty(T, Il, dtype=torch.bfloat16, device="cuda")
    if rows % 256 == 0:
        res_p, a_full_p = tccl.all_gather_gemm(x_sh, wu_r, variant="pair")
        torch.cuda.synchronize()
        ok_p = bool(torch.equal(a_full_p, x_all)) and bool(torch.equal(res_p, res) or (
            (res_p.float() - res.float()).abs() <= res.float().abs() * 2 ** -7 + 1e-2).all())
        report("all_gather_gemm", "tccl_b200 fused (pair)",
               timeit(lambda: tccl.all_gather_gemm(x_sh, wu_r, out=o2, variant="pair")), flops, link, ok_p)
    for cc in [int(v) for v in a.ag_comm_ctas.split(",")]:
        report("all_gather_gemm", f"tccl_b200 fused (single, movers={cc or 'auto'})",
               timeit(lambda: tccl.all_gather_gemm(x_sh, wu_r, out=o2, comm_ctas=cc, variant="single")), flops, link, ok_b)
    gathered = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")

    def unfused_b():
        dist.all_gather_into_tensor(gathered, x_sh)
        torch.matmul(gathered, wu_r.t(), out=o2)
    report("all_gather_gemm", "nccl + cublas", timeit(unfused_b), flops, link, True)

    # ---------------- (c) all-reduce + bias + residual + RMSNorm
    xp = w.empty((T, H), torch.bfloat16)
    xp.copy_(rnd((T, H), 4000 + rank))
    bias, resid, wn = rnd((H,), 1, 0.5), rnd((T, H), 2), rnd((H,), 3)
    y, h_out = tccl.all_reduce_bias_residual_rmsnorm(xp, wn, bias, resid, eps=1e-5, residual_out=True)
    torch.cuda.synchronize()
    from tccl_b200.utils.numerics import allreduce_rmsnorm_check

    s_sum = sum(rnd((T, H), 4000 + r).float() for r in range(W))
    ok_c, _ = allreduce_rmsnorm_check(y, h_out, s_sum, bias, resid, wn, 1e-5, W, w.has_nvls and W > 1)
    del s_sum, h_out
    S = T * H * 2
    link = (S + S // W) if w.has_nvls and W > 2 else 2 * (W - 1) * S // W
    report("allreduce_bias_residual_rmsnorm", "tccl_b200 fused",
           timeit(lambda: tccl.all_reduce_bias_residual_rmsnorm(xp, wn, bias, resid, eps=1e-5)), 0, link, ok_c)
    tmp = xp.clone()

    def unfused_c():
        tmp.copy_(xp)
        dist.all_reduce(tmp)
        h = tmp + bias + resid
        hf = h.float()
        return (hf * torch.rsqrt((hf * hf).mean(-1, keepdim=True) + 1e-5)).to(torch.bfloat16) * wn
    report("allreduce_bias_residual_rmsnorm", "nccl + torch ops", timeit(unfused_c), 0, link, True)

    def unfused_c2():
        tmp.copy_(xp)
        dist.all_reduce(tmp)
        return torch.nn.functional.rms_norm(tmp + bias + resid, (H,), wn, 1e-5)
    report("allreduce_bias_residual_rmsnorm", "nccl + torch rms_norm", timeit(unfused_c2), 0, link, True)

    w.check()
    if a.out and rank == 0:
        os.makedirs(os.path.dirname(a.out) or ".", exist_ok=True)
        with open(a.out, "w") as f:
            for r in rows_out:
                f.write(json.dumps(r) + "\n")
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
