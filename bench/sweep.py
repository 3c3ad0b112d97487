"""Message-size sweeps of the collectives against NCCL (and, when it is
installed under baseline/_ref, the reference's Triton kernels) on the same
GPUs with the same harness: warm-up per size, CUDA events per iteration, p50
of the per-iteration maximum over ranks.

    python -m torch.distributed.run --nproc-per-node 8 bench/sweep.py \
        --collective allreduce --min-bytes 1024 --max-bytes 1073741824 --out gpurun_out/ar8.jsonl

Bus bandwidth uses the nccl-tests factors: all-reduce 2 (W-1)/W on the message
size; all-gather and reduce-scatter (W-1)/W on the total (W shards) size.
Roofline: the bytes each GPU must receive over NVLink divided by the link
bandwidth (--link-gbs, default the measured 770 GB/s per direction).
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
from tccl_b200.utils.timing import max_over_ranks, summarize, time_iters  # noqa: E402


def nvlink_bytes_in(coll, algo, W, S):
    """Bytes one GPU must receive for message size S (per-rank input bytes for
    all-reduce / reduce-scatter, per-rank shard bytes for all-gather)."""
    if W == 1:
        return 0
    if coll == "allreduce":
        if "nvls" in algo:
            return S  # S/W reduced + (W-1)/W S broadcast
        if algo.startswith("oneshot"):
            return (W - 1) * S
        return 2 * (W - 1) * S // W
    if coll == "allgather":
        return (W - 1) * S
    if coll == "reducescatter":
        return (W - 1) * S // W  # egress-bound with NVLS, ingress-bound with P2P: same size
    raise ValueError(coll)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--collective", default="allreduce", choices=["allreduce", "allgather", "reducescatter", "barrier"])
    ap.add_argument("--algos", default="auto")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--min-bytes", type=int, default=1024)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--big-iters", type=int, default=30, help="iterations for messages >= 64 MiB")
    ap.add_argument("--seed", type=int, default=2000)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    ap.add_argument("--nccl", type=int, default=1)
    ap.add_argument("--verify", type=int, default=1)
    ap.add_argument("--graph", type=int, default=0, help="time a CUDA graph of one call (removes host launch time)")
    ap.add_argument("--out", default="")
    a = ap.parse_args()

    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    W = int(os.environ.get("WORLD_SIZE", 1))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", rank=rank, world_size=W, device_id=torch.device("cuda", local_rank))
    w = tccl.init()
    dtype = {"bf16": torch.bfloat16, "fp32": torch.float32}[a.dtype]
    esz = torch.empty(0, dtype=dtype).element_size()
    sync = lambda: dist.barrier()
    rows = []

    def emit(row):
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    if a.collective == "barrier":
        for flavour in ["p2p"] + (["nvls"] if w.has_nvls else []):
            fn = lambda: tccl.barrier(blocks=1, threads=32, rounds=1, flavour=flavour)
            ms = max_over_ranks(time_iters(fn, a.iters, a.warmup, sync=sync))
            emit({"collective": "barrier", "algo": flavour, "world": W, **summarize(ms)})
            fn100 = lambda: tccl.barrier(blocks=1, threads=32, rounds=101, flavour=flavour)
            ms100 = max_over_ranks(time_iters(fn100, a.iters, a.warmup, sync=sync))
            emit({"collective": "barrier_round", "algo": flavour, "world": W,
                  "us_per_round": (summarize(ms100)["p50_us"] - summarize(ms)["p50_us"]) / 100})
        w.check()
        _finish(a, rows, rank)
        return

    max_elems = a.max_bytes // esz
    g = torch.Generator(device="cpu").manual_seed(a.seed + rank)
    n_init = min(max_elems, 1 << 24)
    host = torch.randn(n_init, generator=g).to(dtype)
    if a.collective == "allgather":
        host = (torch.rand(n_init, generator=g) * 2 - 1).to(dtype)
    x_full = w.empty(max_elems, dtype)
    for off in range(0, max_elems, n_init):
        m = min(n_init, max_elems - off)
        x_full[off:off + m].copy_(host[:m])
    out_sym = None
    if a.collective == "allgather":
        out_sym = w.empty(max_elems * W, dtype)
    nccl_out = None

    size = a.max_bytes
    sizes = []
    while size >= a.min_bytes:
        sizes.append(size)
        size //= 2
    for S in sizes:
        n = S // esz
        if a.collective == "reducescatter" and n % (W * (16 // esz)):
            continue
        x = x_full[:n]
        iters = a.big_iters if S >= (64 << 20) else a.iters
        warm = max(3, min(a.warmup, iters))
        if a.algos == "auto":
            if a.collective == "allreduce":
                algos = ["oneshot_p2p"] if S <= (8 << 20) else []
                algos += ["twoshot_p2p"]
                if w.has_nvls:
                    algos += (["oneshot_nvls"] if S <= (8 << 20) else []) + ["twoshot_nvls"]
                algos += ["tree"] if hasattr(tccl, "double_tree_all_reduce") and S >= 4096 else []
            elif a.collective == "allgather":
                algos = ["pull", "push"] + (["push_nvls"] if w.has_nvls else [])
            else:
                algos = ["p2p"] + (["nvls"] if w.has_nvls else [])
        else:
            algos = a.algos.split(",")
        for algo in algos:
            if a.collective == "allreduce":
                if algo.startswith("oneshot"):
                    o = torch.empty_like(x)
                    fn = lambda: tccl.all_reduce(x, out=o, algo=algo)
                else:
                    fn = lambda: tccl.all_reduce(x, inplace=True, algo=algo)
            elif a.collective == "allgather":
                if algo == "pull":
                    o = torch.empty(W * n, dtype=dtype, device="cuda")
                    fn = lambda: tccl.all_gather(x, out=o.view(W, n), algo="pull")
                else:
                    o = out_sym[: W * n].view(W, n)
                    fn = lambda: tccl.all_gather(x, out=o, algo=algo)
            else:
                o = torch.empty(n // W, dtype=dtype, device="cuda")
                fn = lambda: tccl.reduce_scatter(x, out=o, algo=algo)
            run = fn
            if a.graph:
                fn()
                torch.cuda.synchronize()
                dist.barrier()
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    fn()
                run = gr.replay
            ms = max_over_ranks(time_iters(run, iters, warm, sync=sync))
            st = summarize(ms)
            w.check()
            t = st["p50_us"] * 1e-6
            total = S * W if a.collective == "allgather" else S
            factor = (2 * (W - 1) / W) if a.collective == "allreduce" else ((W - 1) / W)
            algbw = S / t / 1e9
            busbw = (total if a.collective != "allreduce" else S) * factor / t / 1e9
            need = nvlink_bytes_in(a.collective, algo, W, S)
            roof_t = need / (a.link_gbs * 1e9) if need else 0.0
            emit({"collective": a.collective, "impl": "tccl_b200", "algo": algo, "world": W, "dtype": a.dtype,
                  "bytes": S, "graph": a.graph, **{k: round(v, 3) if isinstance(v, float) else v for k, v in st.items()},
                  "algbw_gbs": round(algbw, 3), "busbw_gbs": round(busbw, 3),
                  "roofline_frac": round(roof_t / t, 4) if roof_t else None})
            if a.collective == "allreduce" and not algo.startswith("oneshot"):
                # in-place reductions grow the data every iteration: restore it
                for off in range(0, n, n_init):
                    m = min(n_init, n - off)
                    x_full[off:off + m].copy_(host[:m])
        if a.nccl:
            if a.collective == "allreduce":
                y = x.clone()
                fn = lambda: dist.all_reduce(y)
            elif a.collective == "allgather":
                o = torch.empty(W * n, dtype=dtype, device="cuda")
                fn = lambda: dist.all_gather_into_tensor(o, x)
            else:
                o = torch.empty(n // W, dtype=dtype, device="cuda")
                fn = lambda: dist.reduce_scatter_tensor(o, x)
            ms = max_over_ranks(time_iters(fn, iters, warm, sync=sync))
            st = summarize(ms)
            t = st["p50_us"] * 1e-6
            total = S * W if a.collective == "allgather" else S
            factor = (2 * (W - 1) / W) if a.collective == "allreduce" else ((W - 1) / W)
            emit({"collective": a.collective, "impl": "nccl", "algo": "nccl", "world": W, "dtype": a.dtype, "bytes": S,
                  **{k: round(v, 3) if isinstance(v, float) else v for k, v in st.items()},
                  "algbw_gbs": round(S / t / 1e9, 3),
                  "busbw_gbs": round((total if a.collective != "allreduce" else S) * factor / t / 1e9, 3)})
            del fn
    _finish(a, rows, rank)


def _finish(a, rows, rank):
    if a.out and rank == 0:
        os.makedirs(os.path.dirname(a.out) or ".", exist_ok=True)
        with open(a.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
