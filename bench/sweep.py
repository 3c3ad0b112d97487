"""Message-size sweeps of the collectives against NCCL and against the reference's
Triton kernels on the same GPUs with the same harness: every (size, kernel) is
verified once against an fp32 host sum, warmed up, then timed with CUDA events per
iteration; the figure is the p50 of the per-iteration maximum over ranks.

    python -m torch.distributed.run --nproc-per-node 8 bench/sweep.py \
        --collective allreduce,allgather,reducescatter,barrier --ref 1 --out results/sweep8.jsonl

Inputs follow the benchmark configurations: all-reduce up to 1 MiB N(0,1) with
seed 1000 + rank, above that seed 2000 + rank; all-gather and reduce-scatter
U(-1,1) with seed 3000 + rank.  (A 4 Mi-element block is drawn per rank and
repeated through the buffer, so that every rank can rebuild every rank's data.)

Bus bandwidth uses the nccl-tests factors: all-reduce 2 (W-1)/W on the message
size; all-gather and reduce-scatter (W-1)/W on the total (W shards) size.
Roofline: the bytes each GPU must receive over NVLink divided by the link
bandwidth (--link-gbs, default 770 GB/s per direction: what a peer-to-peer
cudaMemcpy reaches on these machines; the nominal figure is 900).
``--graph 1`` times a CUDA graph of one call, which takes the host's launch
path out of small-message latencies; ``--graph 2`` does both for messages up to
4 MiB.  ``--tune-ctas`` repeats the large messages with different CTA counts.

``--ref 1`` adds the reference's own kernels, imported unmodified from
``baseline/_ref`` at run time: ``one_shot_all_reduce`` (triton_one_shot_all_reduce_no_128.py:67-96,
sizes up to 1 MiB), ``one_shot_all_gather`` (triton_all_gather.py:66-95) and
``one_shot_reduce_scatter`` (triton_reduce_scatter.py:95-127, which reads the module globals
``rank`` and ``world_size``: the harness sets them on the imported module).  Each size is
warmed up first, so that Triton's per-size compilation stays outside the timing (the
reference's own loop times it, triton_reduce_scatter.py:213-226); ``--ref-bytes`` limits the
sizes, because every size is a separate compilation.  A leg that raises prints an
``unavailable`` line with the exception.
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

PERIOD = 1 << 22  # elements of the per-rank block that is repeated through the buffers


def nvlink_bytes_in(coll, algo, W, S):
    """Bytes one GPU must receive for message size S (per-rank input bytes for
    all-reduce / reduce-scatter, per-rank shard bytes for all-gather)."""
    if W == 1:
        return 0
    if coll == "allreduce":
        if algo in ("twoshot_nvls", "twoshot_pipe_nvls"):
            return S + S // W  # reduced slice in + every slice broadcast back (own included)
        if algo == "fp8wire":
            return (W - 1) * S // W  # one byte per element, there and back
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


def rank_block(seed, rank, kind, dtype):
    g = torch.Generator(device="cpu").manual_seed(seed + rank)
    t = torch.randn(PERIOD, generator=g) if kind == "normal" else torch.rand(PERIOD, generator=g) * 2 - 1
    return t.to(dtype)


def windows(n, W, span=1 << 14):
    """Element windows to verify: the start of every rank's slice, and the tail."""
    per = -(-n // W)
    starts = sorted({min(q * per, max(0, n - span)) for q in range(W)} | {max(0, n - span)})
    return [(s, min(span, n - s)) for s in starts]


def gather_period(block, start, length):
    idx = (torch.arange(start, start + length) % PERIOD)
    return block[idx]


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
    ap.add_argument("--link-gbs", type=float, default=770.0)
    ap.add_argument("--nccl", type=int, default=1)
    ap.add_argument("--ref", type=int, default=0, help="1: also time the reference's Triton kernels (baseline/_ref)")
    ap.add_argument("--ref-bytes", default="", help="comma list of sizes for the reference legs (default: every 4th size)")
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
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", rank=rank, world_size=W, device_id=dev)
    w = tccl.init()
    dtype = {"bf16": torch.bfloat16, "fp32": torch.float32}[a.dtype]
    esz = torch.empty(0, dtype=dtype).element_size()
    tol = {torch.bfloat16: 2 ** -7, torch.float32: 2e-6}[dtype]
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
    data_colls = [c for c in colls if c != "barrier"]
    blocks = {}      # (seed, kind) -> [every rank's block]
    loaded = [None]  # what x_full holds now

    def load(seed, kind):
        """Fill the symmetric input with this rank's block of (seed, kind), repeated."""
        key = (seed, kind)
        if key not in blocks:
            blocks[key] = [rank_block(seed, r, kind, dtype) for r in range(W)]
        if loaded[0] != key:
            mine = blocks[key][rank].to(dev)
            for off in range(0, max_elems, PERIOD):
                m = min(PERIOD, max_elems - off)
                x_full[off:off + m].copy_(mine[:m])
            loaded[0] = key
        return blocks[key]

    ref_mods = {}
    x_ref = None
    if data_colls:
        x_full = w.empty(max_elems, dtype)
        y_full = w.empty(max_elems, dtype)
    if a.ref and data_colls and dtype == torch.bfloat16 and W > 1:
        try:
            sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
            from torch._C._distributed_c10d import _SymmetricMemory
            from torch.distributed._symmetric_memory import enable_symm_mem_for_group
            import triton_all_gather
            import triton_one_shot_all_reduce_no_128
            import triton_reduce_scatter

            triton_reduce_scatter.rank, triton_reduce_scatter.world_size = rank, W  # the globals its wrapper reads
            ref_mods = {"allreduce": triton_one_shot_all_reduce_no_128, "allgather": triton_all_gather,
                        "reducescatter": triton_reduce_scatter}
            gname = dist.group.WORLD.group_name
            enable_symm_mem_for_group(gname)
            x_ref = _SymmetricMemory.empty_strided_p2p(size=(max_elems,), stride=(1,), dtype=dtype, device=dev,
                                                       group_name=gname)
        except Exception as e:  # noqa: BLE001
            emit({"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:200]}"})
            ref_mods = {}
    sizes = []
    size = a.max_bytes
    while size >= a.min_bytes:
        sizes.append(size)
        size //= 2
    ref_sizes = set(int(v) for v in a.ref_bytes.split(",") if v) or set(sizes[::4])
    tune = [int(v) for v in a.tune_ctas.split(",") if v]

    def check_sum(got, blocks_, n, base=0, partial_roundings=0):
        """`got`: a device tensor holding elements [base, base + len) of the reduced message.
        One rounding of the fp32 sum, plus (double tree) `partial_roundings` roundings of partial
        sums on the way up, each bounded by half an ulp of the sum of magnitudes."""
        worst = 0.0
        for s, ln in windows(got.numel(), W):
            ref = torch.zeros(ln, dtype=torch.float32)
            mag = torch.zeros(ln, dtype=torch.float32)
            for r in range(W):
                v = gather_period(blocks_[r], base + s, ln).float()
                ref += v
                mag += v.abs()
            err = (got[s:s + ln].float().cpu() - ref).abs()
            bound = ref.abs() * tol + mag * (tol / 2) * partial_roundings + 1e-5 * W
            worst = max(worst, float((err / bound).max()))
        return worst

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
            if coll == "allreduce":
                blk = load(1000 if S <= (1 << 20) else 2000, "normal")
            else:
                blk = load(3000, "uniform")
            x = x_full[:n]
            iters = a.big_iters if S * (W if coll == "allgather" else 1) >= (64 << 20) else a.iters
            warm = max(3, min(a.warmup, iters))
            if a.algos == "auto":
                if coll == "allreduce":
                    algos = (["oneshot_p2p"] if S <= (8 << 20) else []) + ["twoshot_p2p"]
                    push_ok = S % 16 == 0 and S <= w.push_max_bytes()
                    algos += ["push_p2p"] if push_ok else []
                    if w.has_nvls:
                        algos += (["oneshot_nvls"] if S <= (8 << 20) else []) + ["twoshot_nvls"]
                        algos += ["push_nvls"] if push_ok else []
                    if W == 2 and S >= (16 << 20):
                        algos += ["twoshot_bulk_p2p"]
                    if S >= (1 << 20):
                        algos += ["twoshot_pipe_nvls" if w.has_nvls and W > 2 else "twoshot_pipe_p2p"]
                    algos += ["tree"] if S >= 4096 else []
                    if a.dtype == "bf16" and S % 4096 == 0 and (1 << 20) <= S <= (64 << 20):
                        algos += ["fp8wire"]  # quantised wire format: not the same arithmetic, reported beside the rest
                elif coll == "allgather":
                    algos = ["pull", "push"] + (["push_nvls"] if w.has_nvls else [])
                else:
                    algos = ["p2p"] + (["nvls"] if w.has_nvls else [])
            else:
                algos = a.algos.split(",")
                if coll == "allreduce":  # drop what does not apply to this size
                    algos = [g_ for g_ in algos if not (g_.startswith("push") and (S % 16 or S > w.push_max_bytes()))
                             and not (g_.startswith("oneshot") and S > (64 << 20)) and not (g_ == "tree" and S % 16)]
            for algo in algos:
                restore = False
                if coll == "allreduce":
                    if algo.startswith("oneshot") or algo.startswith("push"):
                        o = torch.empty_like(x)
                        fn = lambda: tccl.all_reduce(x, out=o, algo=algo)
                        res = lambda: o
                    elif algo == "fp8wire":
                        o = torch.empty_like(x)
                        fn = lambda: tccl.quantized_all_reduce(x, out=o)
                        res = lambda: o
                    elif algo == "tree":
                        fn = lambda: tccl.all_reduce(x, inplace=True, algo="tree")
                        res = lambda: x
                        restore = True  # the in-place reduction grows the data
                    else:
                        y = y_full[:n]
                        fn = lambda: tccl.all_reduce(x, out=y, algo=algo)
                        res = lambda: y
                    fn()
                    torch.cuda.synchronize()
                    # fp8 wire: two roundings to 3 mantissa bits of values up to a chunk's maximum (<= ~5 sigma)
                    pr = max(1, W.bit_length()) if algo == "tree" else (64 if algo == "fp8wire" else 0)
                    worst = check_sum(res(), blk, n, partial_roundings=pr)
                elif coll == "allgather":
                    if algo == "pull":
                        o = torch.empty(W * n, dtype=dtype, device=dev)
                        fn = lambda: tccl.all_gather(x, out=o.view(W, n), algo="pull")
                    else:
                        o = y_full[: W * n]
                        fn = lambda: tccl.all_gather(x, out=o.view(W, n), algo=algo)
                    o.zero_()
                    fn()
                    torch.cuda.synchronize()
                    worst = 0.0
                    for r in range(W):
                        for s, ln in windows(n, 1):
                            same = torch.equal(o[r * n + s:r * n + s + ln].cpu(), gather_period(blk[r], s, ln))
                            worst = max(worst, 0.0 if same else 2.0)
                else:
                    o = torch.empty(n // W, dtype=dtype, device=dev)
                    fn = lambda: tccl.reduce_scatter(x, out=o, algo=algo)
                    fn()
                    torch.cuda.synchronize()
                    worst = check_sum(o, blk, n, base=rank * (n // W))
                if restore:
                    loaded[0] = None
                    load(1000 if S <= (1 << 20) else 2000, "normal")
                bad = torch.tensor([worst], device=dev)
                dist.all_reduce(bad, op=dist.ReduceOp.MAX)
                verified = float(bad.item()) <= 1.0
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
                          "bytes": S, "graph": graph, "ctas": ctas, "verified": verified,
                          **{k: round(v, 3) if isinstance(v, float) else v for k, v in st.items()},
                          "algbw_gbs": round(S / t / 1e9, 3), "busbw_gbs": round(total * factor / t / 1e9, 3),
                          "algo_roofline_frac": round(need / (a.link_gbs * 1e9) / t, 4) if need else None,
                          "roofline_frac": round(best / (a.link_gbs * 1e9) / t, 4) if best else None})
                    if restore:
                        loaded[0] = None
                        load(1000 if S <= (1 << 20) else 2000, "normal")
                if tune:
                    w.reconfigure(max_ctas=0)
            factor = (2 * (W - 1) / W) if coll == "allreduce" else ((W - 1) / W)
            total = S * W if coll == "allgather" else S
            if a.nccl:
                if coll == "allreduce":
                    yy = y_full[:n]
                    yy.zero_()  # in place: zeros stay finite over any number of iterations
                    fn = lambda: dist.all_reduce(yy)
                elif coll == "allgather":
                    o = torch.empty(W * n, dtype=dtype, device=dev)
                    fn = lambda: dist.all_gather_into_tensor(o, x)
                else:
                    o = torch.empty(n // W, dtype=dtype, device=dev)
                    fn = lambda: dist.reduce_scatter_tensor(o, x)
                for graph in ([0, 1] if a.graph == 2 and S <= (4 << 20) else [a.graph if a.graph < 2 else 0]):
                    st = measure(fn, iters, warm, graph)
                    t = st["p50_us"] * 1e-6
                    best = best_possible_bytes_in(coll, W, S, True)
                    emit({"collective": coll, "impl": "nccl", "algo": "nccl", "world": W, "dtype": a.dtype, "bytes": S,
                          "graph": graph, **{k: round(v, 3) if isinstance(v, float) else v for k, v in st.items()},
                          "algbw_gbs": round(S / t / 1e9, 3), "busbw_gbs": round(total * factor / t / 1e9, 3),
                          "roofline_frac": round(best / (a.link_gbs * 1e9) / t, 4) if best else None})
            mod = ref_mods.get(coll)
            size_key = S * W if coll == "allgather" else S
            if mod is not None and size_key in ref_sizes and not (coll == "allreduce" and S > (1 << 20)):
                try:
                    xr = x_ref[:n]
                    xr.copy_(x)
                    torch.cuda.synchronize()
                    dist.barrier()
                    if coll == "allreduce":
                        if n % 4:
                            raise ValueError("the reference needs numel % 4 == 0")
                        fn = lambda: mod.one_shot_all_reduce(xr)
                    elif coll == "allgather":
                        fn = lambda: mod.one_shot_all_gather(xr, W)
                    else:
                        fn = lambda: mod.one_shot_reduce_scatter(xr)
                    out_r = fn()  # compiles this size
                    torch.cuda.synchronize()
                    dist.barrier()
                    if coll == "allgather":
                        ok = all(torch.equal(out_r[r, :1 << 12].cpu(), gather_period(blk[r], 0, min(n, 1 << 12))) for r in range(W))
                    else:
                        base = rank * (n // W) if coll == "reducescatter" else 0
                        ln = min(out_r.numel(), 1 << 14)
                        ref = torch.zeros(ln, dtype=torch.float32)
                        mag = torch.zeros(ln, dtype=torch.float32)
                        for r in range(W):
                            ref += gather_period(blk[r], base, ln).float()
                            mag += ref.abs()
                        # the reference adds in bf16, rank after rank: half an ulp of every running sum
                        ok = bool(((out_r[:ln].float().cpu() - ref).abs() <= mag * 2 ** -8 * 1.01 + 1e-5 * W).all())
                    st = summarize(max_over_ranks(time_iters(fn, iters, warm, sync=sync)))
                    t = st["p50_us"] * 1e-6
                    emit({"collective": coll, "impl": "reference_triton", "algo": "one_shot", "world": W, "dtype": a.dtype,
                          "bytes": S, "graph": 0, "verified": ok,
                          **{k: round(v, 3) if isinstance(v, float) else v for k, v in st.items()},
                          "algbw_gbs": round(S / t / 1e9, 3), "busbw_gbs": round(total * factor / t / 1e9, 3)})
                except Exception as e:  # noqa: BLE001
                    emit({"collective": coll, "impl": "reference_triton", "bytes": S, "world": W,
                          "unavailable": f"{type(e).__name__}: {str(e)[:200]}"})
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
