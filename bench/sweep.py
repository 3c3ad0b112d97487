"""Message-size sweeps of the collectives against NCCL on the same GPUs with
the same harness: warm-up per size, CUDA events per iteration, p50 of the
per-iteration maximum over ranks.

    python -m torch.distributed.run --nproc-per-node 8 bench/sweep.py \
        --collective allreduce,allgather,reducescatter,barrier --out results/sweep8.jsonl

Bus bandwidth uses the nccl-tests factors: all-reduce 2 (W-1)/W on the message
size; all-gather and reduce-scatter (W-1)/W on the total (W shards) size.
Roofline: the bytes each GPU must receive over NVLink divided by the link
bandwidth (--link-gbs, default the measured 770 GB/s per direction).
``--graph 1`` times a CUDA graph of one call, which takes the host's launch
path out of small-message latencies; ``--graph 2`` does both for messages up to
4 MiB.  ``--tune-ctas`` repeats the large messages with different CTA counts.
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
        if algo == "twoshot_nvls":
            return S + S // W  # reduced slice in + every slice broadcast back (own included)
        if algo.startswith("push"):
            return (W - 1) * S
        if algo == "oneshot_nvls":
            return S
        if algo == "oneshot_p2p":
            return (W - 1) * S
        if algo == "tree":
            return 2 * S  # interior in one tree (2 children up + 1 down on S/2), leaf in the other
        return 2 * (W - 1) * S // W
    if coll == "allgather":
        return (W - 1) * S
    if coll == "reducescatter":
        return (W - 1) * S // W
    raise ValueError(coll)


def best_possible_bytes_in(coll, W, S, nvls):
    """Roofline denominator: the least any algorithm here must receive."""
    if W == 1:
        return 0
    if coll == "allreduce":
        return S if nvls else 2 * (W - 1) * S // W
    if coll == "allgather":
        return (W - 1) * S
    return (W - 1) * S // W


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--collective", default="allreduce")
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
    ap.add_argument("--graph", type=int, default=0)
    ap.add_argument("--tune-ctas", default="")
    ap.add_argument("--tune-min-bytes", type=int, default=64 << 20)
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

    def measure(fn, iters, warm, graph):
        run = fn
        if graph:
            fn()
            torch.cuda.synchronize()
            dist.barrier()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                fn()
            run = gr.replay
        st = summarize(max_over_ranks(time_iters(run, iters, warm, sync=sync)))
        w.check()
        return st

    colls = a.collective.split(",")
    if "barrier" in colls:
        for flavour in ["p2p"] + (["nvls"] if w.has_nvls else []):
            for graph in ([0, 1] if a.graph == 2 else [a.graph]):
                st1 = measure(lambda: tccl.barrier(blocks=1, threads=32, rounds=1, flavour=flavour), a.iters, a.warmup, graph)
                st101 = measure(lambda: tccl.barrier(blocks=1, threads=32, rounds=101, flavour=flavour), a.iters, a.warmup, graph)
                emit({"collective": "barrier", "algo": flavour, "world": W, "graph": graph,
                      "p50_us": round(st1["p50_us"], 3), "us_per_round": round((st101["p50_us"] - st1["p50_us"]) / 100, 3)})

    max_elems = a.max_bytes // esz
    n_init = min(max_elems, 1 << 24)
    data_colls = [c for c in colls if c != "barrier"]
    if data_colls:
        g = torch.Generator(device="cpu").manual_seed(a.seed + rank)
        host = torch.randn(n_init, generator=g).to(dtype)
        x_full = w.empty(max_elems, dtype)
        y_full = w.empty(max_elems, dtype)
        for off in range(0, max_elems, n_init):
            m = min(n_init, max_elems - off)
            x_full[off:off + m].copy_(host[:m])
    sizes = []
    size = a.max_bytes
    while size >= a.min_bytes:
        sizes.append(size)
        size //= 2
    tune = [int(v) for v in a.tune_ctas.split(",") if v]

    for coll in data_colls:
        for S in sizes:
            n = S // esz
            if coll == "reducescatter" and n % (W * (16 // esz)):
                continue
            if coll == "allgather":
                n = n // W  # sweep the gathered size so that the symmetric output fits max-bytes
                if n < 8:
                    continue
                S = n * esz
            x = x_full[:n]
            iters = a.big_iters if S * (W if coll == "allgather" else 1) >= (64 << 20) else a.iters
            warm = max(3, min(a.warmup, iters))
            if a.algos == "auto":
                if coll == "allreduce":
                    algos = (["oneshot_p2p"] if S <= (8 << 20) else []) + ["twoshot_p2p"]
                    push_ok = S % 16 == 0 and 2 * W * S <= w.ll_bytes
                    algos += ["push_p2p"] if push_ok else []
                    if w.has_nvls:
                        algos += (["oneshot_nvls"] if S <= (8 << 20) else []) + ["twoshot_nvls"]
                        algos += ["push_nvls"] if push_ok else []
                    algos += ["tree"] if S >= 4096 else []
                elif coll == "allgather":
                    algos = ["pull", "push"] + (["push_nvls"] if w.has_nvls else [])
                else:
                    algos = ["p2p"] + (["nvls"] if w.has_nvls else [])
            else:
                algos = a.algos.split(",")
            for algo in algos:
                if coll == "allreduce":
                    if algo.startswith("oneshot") or algo.startswith("push"):
                        o = torch.empty_like(x)
                        fn = lambda: tccl.all_reduce(x, out=o, algo=algo)
                    elif algo == "tree":
                        fn = lambda: tccl.all_reduce(x, inplace=True, algo="tree")
                    else:
                        y = y_full[:n]
                        fn = lambda: tccl.all_reduce(x, out=y, algo=algo)
                elif coll == "allgather":
                    if algo == "pull":
                        o = torch.empty(W * n, dtype=dtype, device="cuda")
                        fn = lambda: tccl.all_gather(x, out=o.view(W, n), algo="pull")
                    else:
                        o = y_full[: W * n].view(W, n)
                        fn = lambda: tccl.all_gather(x, out=o, algo=algo)
                else:
                    o = torch.empty(n // W, dtype=dtype, device="cuda")
                    fn = lambda: tccl.reduce_scatter(x, out=o, algo=algo)
                variants = [(None, g_) for g_ in ([0, 1] if a.graph == 2 and S <= (4 << 20) else [a.graph if a.graph < 2 else 0])]
                if tune and S >= a.tune_min_bytes and algo != "tree":
                    variants = [(c, 0) for c in tune]
                for ctas, graph in variants:
                    if ctas is not None:
                        w.reconfigure(max_ctas=ctas)
                    st = measure(fn, iters, warm, graph)
                    t = st["p50_us"] * 1e-6
                    factor = (2 * (W - 1) / W) if coll == "allreduce" else ((W - 1) / W)
                    total = S * W if coll == "allgather" else S
                    need = nvlink_bytes_in(coll, algo, W, S)
                    best = best_possible_bytes_in(coll, W, S, w.has_nvls)
                    emit({"collective": coll, "impl": "tccl_b200", "algo": algo, "world": W, "dtype": a.dtype,
                          "bytes": S, "graph": graph, "ctas": ctas,
                          **{k: round(v, 3) if isinstance(v, float) else v for k, v in st.items()},
                          "algbw_gbs": round(S / t / 1e9, 3), "busbw_gbs": round(total * factor / t / 1e9, 3),
                          "algo_roofline_frac": round(need / (a.link_gbs * 1e9) / t, 4) if need else None,
                          "roofline_frac": round(best / (a.link_gbs * 1e9) / t, 4) if best else None})
                    if algo == "tree":  # the in-place reduction grows the data: restore it
                        for off in range(0, n, n_init):
                            m = min(n_init, n - off)
                            x_full[off:off + m].copy_(host[:m])
                if tune:
                    w.reconfigure(max_ctas=0)
            if a.nccl:
                if coll == "allreduce":
                    yy = y_full[:n]
                    yy.copy_(x)
                    fn = lambda: dist.all_reduce(yy)
                elif coll == "allgather":
                    o = torch.empty(W * n, dtype=dtype, device="cuda")
                    fn = lambda: dist.all_gather_into_tensor(o, x)
                else:
                    o = torch.empty(n // W, dtype=dtype, device="cuda")
                    fn = lambda: dist.reduce_scatter_tensor(o, x)
                for graph in ([0, 1] if a.graph == 2 and S <= (4 << 20) else [a.graph if a.graph < 2 else 0]):
                    st = measure(fn, iters, warm, graph)
                    t = st["p50_us"] * 1e-6
                    factor = (2 * (W - 1) / W) if coll == "allreduce" else ((W - 1) / W)
                    total = S * W if coll == "allgather" else S
                    best = best_possible_bytes_in(coll, W, S, True)
                    emit({"collective": coll, "impl": "nccl", "algo": "nccl", "world": W, "dtype": a.dtype, "bytes": S,
                          "graph": graph, **{k: round(v, 3) if isinstance(v, float) else v for k, v in st.items()},
                          "algbw_gbs": round(S / t / 1e9, 3), "busbw_gbs": round(total * factor / t / 1e9, 3),
                          "roofline_frac": round(best / (a.link_gbs * 1e9) / t, 4) if best else None})
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
