"""Multi-GPU correctness worker: one process per GPU, started by
``torch.distributed.run`` from tests/test_multigpu.py (or by hand).  Every rank
regenerates all ranks' seeded inputs on the CPU, so each rank checks its own
result against an fp32 host sum without extra communication.  Prints one JSON
line per rank-0 summary and exits non-zero on any failure."""
import json
import os
import sys
import traceback

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import tccl_b200 as tccl  # noqa: E402
from tccl_b200.utils.numerics import allreduce_rmsnorm_check  # noqa: E402

TOL = {torch.bfloat16: 2 ** -8, torch.float16: 2 ** -11, torch.float32: 1e-6}


def seeded(n, dtype, seed, kind="normal"):
    g = torch.Generator(device="cpu").manual_seed(seed)
    t = torch.randn(n, generator=g) if kind == "normal" else torch.rand(n, generator=g) * 2 - 1
    return t.to(dtype)


NOTES = []


def close(out, ref, dtype, W, ulps=1.0):
    """|out - ref| within `ulps` half-ulps of one rounding of the fp32 sum."""
    err = (out.float().cpu() - ref).abs()
    ok = bool((err <= ref.abs() * TOL[dtype] * ulps + 1e-6 * W).all())
    if not ok:
        rel = (err / ref.abs().clamp_min(1e-3)).max().item()
        NOTES.append(f"max rel err {rel:.3e} ({rel / TOL[dtype]:.2f} x tol), dtype {dtype}")
    return ok


def main():
    rank = int(os.environ["RANK"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    W = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    w = tccl.init()
    failures, ran = [], []

    def case(name, fn):
        try:
            ok = fn()
            torch.cuda.synchronize()
            w.check()
            ran.append(name)
            if ok is False:
                failures.append(name)
        except Exception as e:  # noqa: BLE001
            failures.append(f"{name}: {type(e).__name__}: {e}")
            traceback.print_exc()

    nvls = w.has_nvls
    ar_algos = ["oneshot_p2p", "twoshot_p2p", "twoshot_pipe_p2p", "twoshot_bulk_p2p"] + (
        ["oneshot_nvls", "twoshot_nvls", "twoshot_pipe_nvls"] if nvls else [])
    push_algos = ["push_p2p"] + (["push_nvls"] if nvls else [])

    # barriers
    case("barrier_p2p", lambda: tccl.barrier(blocks=8, threads=64, rounds=20))
    if nvls:
        case("barrier_nvls", lambda: tccl.barrier(blocks=8, threads=64, rounds=20, flavour="nvls"))

    def cas():
        t = w.empty(4096, torch.int32)
        t.zero_()
        h = w.handle(t)
        for _ in range(3):
            tccl.barrier_test(h, blocks=32, threads=128)
        torch.cuda.synchronize()
        pad = h.get_signal_pad(w.rank, (32 * W,), dtype=torch.int32)
        return int(pad.abs().sum()) == 0
    case("barrier_cas_on_torch_pads", cas)

    for dtype in (torch.bfloat16, torch.float32):
        for n in (8, 4096 + 8, 100003, 1 << 20, (1 << 24) + 16):
            xs = [seeded(n, dtype, 2000 + r) for r in range(W)]
            ref = torch.stack([x.float() for x in xs]).sum(0)
            x = w.empty(n, dtype)
            for algo in ar_algos:
                def ar(algo=algo):
                    x.copy_(xs[rank])
                    # the switch's final bf16 conversion is not round-to-nearest: allow one full ulp
                    ulps = 2.0 if algo.endswith("nvls") else 1.0
                    if algo.startswith("oneshot"):
                        out = tccl.all_reduce(x, algo=algo)
                        return close(out, ref, dtype, W, ulps) and torch.equal(x.cpu(), xs[rank])
                    tccl.all_reduce(x, inplace=True, algo=algo)
                    return close(x, ref, dtype, W, ulps)
                case(f"allreduce/{algo}/{dtype}/{n}", ar)
            if n * x.element_size() % 16 == 0 and n * x.element_size() <= w.push_max_bytes():
                for algo in push_algos:
                    def push_ar(algo=algo):
                        ok = True
                        plain = xs[rank].cuda()  # ordinary (non symmetric) memory
                        for _ in range(3):
                            out = tccl.all_reduce(plain, algo=algo)
                            ok = ok and close(out, ref, dtype, W)
                        return ok
                    case(f"allreduce/{algo}/{dtype}/{n}", push_ar)
            if n % (W * 8) == 0:
                for algo in ["p2p"] + (["nvls"] if nvls else []):
                    def rs(algo=algo):
                        x.copy_(xs[rank])
                        out = tccl.reduce_scatter(x, algo=algo)
                        per = n // W
                        return close(out, ref[rank * per:(rank + 1) * per], dtype, W, 2.0 if algo == "nvls" else 1.0)
                    case(f"reducescatter/{algo}/{dtype}/{n}", rs)

    for n in (8, 1003, 1 << 16, (1 << 22) + 8):
        xs = [seeded(n, torch.bfloat16, 3000 + r, "uniform") for r in range(W)]
        ref = torch.stack(xs)
        x = w.empty(n, torch.bfloat16)
        x.copy_(xs[rank])

        def pull():
            return torch.equal(tccl.one_shot_all_gather(x, W).cpu(), ref)
        case(f"allgather/pull/{n}", pull)
        if n % 8 == 0:
            out = w.empty((W, n), torch.bfloat16)
            for algo in ["push"] + (["push_nvls"] if nvls else []):
                def push(algo=algo):
                    out.zero_()
                    tccl.all_gather(x, out=out, algo=algo)
                    return torch.equal(out.cpu(), ref)
                case(f"allgather/{algo}/{n}", push)

    # fused compute + collective kernels against fp32 references computed on this GPU
    def rnd(shape, seed, scale=1.0):
        g = torch.Generator(device="cpu").manual_seed(seed)
        return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).cuda()

    M, N, Kr = 128 * W * 2, 512, 448

    def gemm_rs():
        a, bt = rnd((M, Kr), 4000 + rank), rnd((N, Kr), 5000 + rank, 0.02)
        ok = True
        for _ in range(2):
            out = tccl.gemm_reduce_scatter(a, bt)
            torch.cuda.synchronize()
            rows = M // W
            ref = sum(rnd((M, Kr), 4000 + r)[rank * rows:(rank + 1) * rows].float() @ rnd((N, Kr), 5000 + r, 0.02).float().t()
                      for r in range(W))
            ok = ok and bool(((out.float() - ref).abs() <= ref.abs() * 2 ** -7 + 0.02 * W).all())
        return ok
    case("fused/gemm_reduce_scatter", gemm_rs)

    def ag_gemm():
        rows = M // W
        sh, bt = rnd((rows, 512), 4000 + rank), rnd((768, 512), 6000 + rank, 0.02)
        ok = True
        for _ in range(2):
            out, a_full = tccl.all_gather_gemm(sh, bt)
            torch.cuda.synchronize()
            x_all = torch.cat([rnd((rows, 512), 4000 + r) for r in range(W)])
            ref = x_all.float() @ bt.float().t()
            ok = ok and bool(((out.float() - ref).abs() <= ref.abs() * 2 ** -8 + 1e-2).all()) and torch.equal(a_full, x_all)
        return ok
    case("fused/all_gather_gemm", ag_gemm)

    for algo in ["p2p"] + (["nvls"] if nvls else []):
        def arn(algo=algo):
            T, H = 67 * W, 4096
            xp = w.empty((T, H), torch.bfloat16)
            xp.copy_(rnd((T, H), 4000 + rank))
            bias, resid, wn = rnd((H,), 1, 0.5), rnd((T, H), 2), rnd((H,), 3)
            y, h_out = tccl.all_reduce_bias_residual_rmsnorm(xp, wn, bias, resid, eps=1e-5, residual_out=True, algo=algo)
            torch.cuda.synchronize()
            s_sum = sum(rnd((T, H), 4000 + r).float() for r in range(W))
            # element-wise bounds that follow from the arithmetic (utils/numerics.py)
            ok, worst = allreduce_rmsnorm_check(y, h_out, s_sum, bias, resid, wn, 1e-5, W, algo == "nvls")
            if not ok:
                NOTES.append(f"rmsnorm/{algo}: worst err/bound of the pre-norm sum {worst:.3f}")
            return ok
        case(f"fused/allreduce_rmsnorm/{algo}", arn)

    def tree():
        ok = True
        for n in (4096, (1 << 20) + 64, 1 << 24):
            xs = [seeded(n, torch.bfloat16, 2000 + r) for r in range(W)]
            ref = torch.stack([x.float() for x in xs]).sum(0)
            x = w.empty(n, torch.bfloat16)
            x.copy_(xs[rank])
            out = tccl.double_tree_all_reduce(x)
            torch.cuda.synchronize()
            err = (out.float().cpu() - ref).abs()
            ok = ok and bool((err <= ref.abs() * 2 ** -8 * 4 + 0.08).all()) and torch.equal(x.cpu(), xs[rank])
            tccl.double_tree_all_reduce(x, inplace=True)
            torch.cuda.synchronize()
            ok = ok and torch.equal(x, out)  # same tree, same order of additions: the same bits
        return ok
    case("allreduce/tree", tree)

    def tree_small():
        """Small messages: the tree whose data lines carry their own flags; many calls in a row, sizes
        changing, no synchronisation in between; in place and out of place."""
        ok = True
        outs = []
        for it in range(40):
            n = [8, 4096, 1 << 15, 1 << 16, 1000 * 8][it % 5]  # up to 256 KiB: nothing has to be symmetric
            xs = [seeded(n, torch.float32, 7000 + 16 * it + r) for r in range(W)]
            x = xs[rank].cuda()
            if it % 2:
                tccl.double_tree_all_reduce(x, inplace=True)
                outs.append((x, torch.stack(xs).sum(0)))
            else:
                outs.append((tccl.double_tree_all_reduce(x), torch.stack(xs).sum(0)))
        torch.cuda.synchronize()
        for o, ref in outs:
            ok = ok and bool(((o.cpu() - ref).abs() <= ref.abs() * 1e-5 + 1e-5).all())
        return ok
    case("allreduce/tree_small_messages", tree_small)

    def quantized():
        """fp8 on the wire: every rank gets the same bits, within two e4m3 roundings of the fp32 sum."""
        ok = True
        for n in (2048, 2048 * 37, 2048 * 4096):
            xs = [seeded(n, torch.bfloat16, 8000 + r) for r in range(W)]
            ref = torch.stack([x.float() for x in xs]).sum(0)
            x = xs[rank].cuda()
            for _ in range(2):
                out = tccl.quantized_all_reduce(x)
            torch.cuda.synchronize()
            cmax = torch.stack([t.float().view(-1, 2048).abs().amax(1) for t in xs]).sum(0)
            bound = ((cmax + ref.view(-1, 2048).abs().amax(1)) * 2 ** -4 * 1.05).unsqueeze(1).expand(-1, 2048).reshape(-1) + 1e-6
            ok = ok and bool(((out.float().cpu() - ref).abs() <= bound).all())
            gathered = [torch.empty_like(out) for _ in range(W)]
            dist.all_gather(gathered, out)
            ok = ok and all(torch.equal(g, out) for g in gathered)
        return ok
    case("allreduce/fp8_wire", quantized)

    def auto_paths():
        """`algo="auto"` end to end: push (small), one-shot (medium), staged two-shot (large, ordinary
        destination), in-place two-shot (large, symmetric)."""
        ok = True
        for n in (1024, 1 << 17, (1 << 22) + 8):
            xs = [seeded(n, torch.bfloat16, 2000 + r) for r in range(W)]
            ref = torch.stack([x.float() for x in xs]).sum(0)
            x = w.empty(n, torch.bfloat16)
            x.copy_(xs[rank])
            out = tccl.all_reduce(x)
            ok = ok and close(out, ref, torch.bfloat16, W, 2.0) and torch.equal(x.cpu(), xs[rank])
            tccl.all_reduce(x, inplace=True)
            ok = ok and close(x, ref, torch.bfloat16, W, 2.0)
        return ok
    case("allreduce/auto", auto_paths)

    def graph_replay():
        """A captured collective replays correctly (all sync state lives on the device)."""
        n = 1 << 14
        x = w.empty(n, torch.float32)
        o = torch.empty_like(x)
        x.fill_(float(rank + 1))
        algos = ["oneshot_p2p", "push_p2p"] + (["twoshot_nvls"] if nvls else ["twoshot_p2p"])
        ok = True
        for algo in algos:
            y = w.empty(n, torch.float32) if algo.startswith("twoshot") else o
            fn = (lambda: tccl.all_reduce(x, out=y, algo=algo))
            fn()
            torch.cuda.synchronize()
            dist.barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            for it in range(5):
                x.fill_(float((rank + 1) * (it + 1)))
                g.replay()
                torch.cuda.synchronize()
                ok = ok and bool((y == float((it + 1) * W * (W + 1) // 2)).all())
        return ok
    case("cuda_graph_replay", graph_replay)

    # back-to-back stress with changing data (WAR/RAW hazards)
    def stress():
        n = 4096
        x = w.empty(n, torch.float32)
        ok = True
        algos = ar_algos + push_algos + ["tree"]
        for it in range(300):
            x.fill_(float(it * (rank + 1)))
            algo = algos[it % len(algos)]
            if algo.startswith("oneshot") or algo.startswith("push"):
                o = tccl.all_reduce(x, algo=algo)
            else:
                o = tccl.all_reduce(x, inplace=True, algo=algo)
            if it % 50 >= 40:
                ok = ok and bool((o == float(it * W * (W + 1) // 2)).all())
        return ok
    case("stress", stress)

    def push_mixed_sizes():
        """Push all-reduces of 64 KiB, 32 KiB and 1 KiB in turn (different grids too), 1000 calls,
        no host synchronisation in between, ranks free to drift a call apart."""
        sizes = [s for s in (16384, 8192, 256) if s * 4 <= w.push_max_bytes()]
        bufs = {n: torch.empty(n, dtype=torch.float32, device="cuda") for n in sizes}
        ok = True
        for algo in push_algos:
            checks = []
            for it in range(1000):
                n = sizes[it % len(sizes)]
                bufs[n].fill_(float((it % 97) * (rank + 1)))
                o = tccl.all_reduce(bufs[n], algo=algo)
                if it % 40 >= 37:
                    checks.append((o, float((it % 97) * W * (W + 1) // 2)))
            torch.cuda.synchronize()
            ok = ok and all(bool((o == want).all()) for o, want in checks)
        return ok
    case("push_mixed_sizes", push_mixed_sizes)

    def tree_changing_sizes():
        """Tree all-reduces back to back with changing size: no barrier separates the calls."""
        ok = True
        outs = []
        for it in range(12):
            n = [1 << 16, 4096, (1 << 20) + 64, 8][it % 4]
            xs = [seeded(n, torch.float32, 5000 + 16 * it + r) for r in range(W)]
            x = xs[rank].cuda()  # ordinary memory: only the in-place form needs a symmetric input
            outs.append((tccl.double_tree_all_reduce(x), torch.stack(xs).sum(0)))
        torch.cuda.synchronize()
        for o, ref in outs:
            ok = ok and bool(((o.cpu() - ref).abs() <= ref.abs() * 1e-5 + 1e-5).all())
        return ok
    case("allreduce/tree_changing_sizes", tree_changing_sizes)

    bad = torch.tensor([len(failures)], device="cuda")
    dist.all_reduce(bad)
    if rank == 0:
        print(json.dumps({"ran": ran}), flush=True)  # the record of what this run covered
        print(json.dumps({"world": W, "nvls": nvls, "cases": len(ran), "failures_rank0": failures, "notes": NOTES[:6],
                          "total_failures": int(bad.item())}), flush=True)
    elif failures:
        print(f"[rank {rank}] failures: {failures}", flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(1 if int(bad.item()) else 0)


if __name__ == "__main__":
    main()
