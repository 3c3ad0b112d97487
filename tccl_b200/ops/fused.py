"""Fused compute + collective ops for tensor parallelism (the "extensible
collectives" the reference names as its motivation — ``presentation.pdf``, slide 4
— but does not implement): GEMM -> reduce-scatter, all-gather -> GEMM, and all-reduce + bias +
residual + RMSNorm.  Each is ONE kernel in which the tensor-core tiles
(tcgen05 / TMEM, fed by TMA from local memory) and the peer traffic (P2P or
NVLS stores / loads over NVLink) overlap tile by tile.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from ..parallel.world import WorldBase
from ..utils import lib as L
from ._common import K, check_sym_tensor, dtype_code, get_world

__all__ = ["gemm_reduce_scatter", "all_gather_gemm", "all_reduce_bias_residual_rmsnorm", "pack_gate_up",
           "ag_pair_schedule"]


def _locals(w: WorldBase, x):
    """Per-rank local tensors of an ordinary (non symmetric) argument: a tensor in
    a real world, a list/EmuTensor of W tensors in an emulated one."""
    if w.plans is not None:  # a real world drives exactly one rank
        return {w.local_ranks[0]: x}
    return {r: x[r] for r in w.local_ranks}


def _trace_ptr(w: WorldBase, trace, r: int, grid: int) -> int:
    """``trace``: an int64 CUDA tensor of at least ``grid * 64`` words (a list of them when
    emulated) that receives per-tile %globaltimer stamps; None = no tracing."""
    if trace is None:
        return 0
    t = trace if w.plans is not None else trace[r]
    if t.dtype != torch.int64 or t.numel() < grid * 64 or not t.is_cuda:
        raise ValueError(f"trace must be an int64 CUDA tensor of >= {grid * 64} words")
    return t.data_ptr()


def _gemm_ctas(w: WorldBase, pairs: bool = False) -> int:
    n = w.config.max_ctas or w.num_sms()
    if w.plans is None:  # emulated ranks share one GPU and each CTA takes a whole SM
        n = max(1, w.num_sms() // w.world_size)
    return max(2, n & ~1) if pairs else n


def _stage_handoff(w: WorldBase, user: str) -> bool:
    """Whether a kernel that runs without an entry barrier must take one this time: the staging
    area was last used by a different kernel (every rank sees the same sequence of calls)."""
    last = w.__dict__.get("_stage_user")
    w.__dict__["_stage_user"] = user
    return last != user


def gemm_reduce_scatter(a, bt, out=None, *, trace=None, variant: str = "auto", world: Optional[WorldBase] = None):
    """``out_r = rows r of sum_ranks (a_rank @ bt_rank.T)`` — tensor-parallel
    down-projection fused with the reduce-scatter over token rows.

    ``a``: this rank's ``[M, K_r]`` activations (its slice of the contraction
    dimension), ``bt``: its ``[N, K_r]`` weight slice (``nn.Linear`` layout), both
    bf16.  Returns this rank's ``[M / W, N]`` rows.  ``M % (128 W) == 0`` and
    ``N % 256 == 0``.  Inputs and output are ordinary tensors; the partial tiles
    travel through the communicator's symmetric staging area.

    ``variant``: ``"pair"`` = 256 x 256 tiles on pairs of SMs, the reduction overlapped with the
    mainloop, no entry barrier (needs ``M % (256 W) == 0`` and twice the staging space);
    ``"single"`` = 128 x 256 single-CTA tiles; ``"auto"`` = pair when the shape allows."""
    w = get_world(world)
    W = w.world_size
    As, Bs = _locals(w, a), _locals(w, bt)
    a0, b0 = As[w.local_ranks[0]], Bs[w.local_ranks[0]]
    if a0.dtype != torch.bfloat16 or b0.dtype != torch.bfloat16:
        raise TypeError("gemm_reduce_scatter takes bfloat16 operands")
    M, Kr = a0.shape
    N = b0.shape[0]
    if b0.shape[1] != Kr:
        raise ValueError("a is [M, K], bt is [N, K]")
    if M % (W * 128) or N % 256 or Kr % 8:
        raise ValueError(f"need M % {W * 128} == 0, N % 256 == 0, K % 8 == 0 (got M={M}, N={N}, K={Kr})")
    lib = L.lib()
    for f in ("tccl_gemm_rs_stage_bytes", "tccl_gemm_rs_param_bytes", "tccl_gemm_rs_pair_stage_bytes",
              "tccl_gemm_rs_pair_param_bytes"):
        getattr(lib, f).restype = C.c_uint64
    stage_bytes = (w.config.stage_mb << 20) - w.ll_bytes
    if variant not in ("auto", "pair", "single"):
        raise ValueError("variant must be 'auto', 'pair' or 'single'")
    pair_ok = M % (W * 256) == 0 and lib.tccl_gemm_rs_pair_stage_bytes(M, N, W) <= stage_bytes
    if variant == "pair" and not pair_ok:
        raise ValueError(f"the pair kernel needs M % {W * 256} == 0 and "
                         f"{lib.tccl_gemm_rs_pair_stage_bytes(M, N, W) >> 20} MiB of staging area")
    pair = pair_ok and variant != "single"
    need = lib.tccl_gemm_rs_pair_stage_bytes(M, N, W) if pair else lib.tccl_gemm_rs_stage_bytes(M, N, W)
    if need > stage_bytes:
        raise ValueError(f"staging area too small: need {need >> 20} MiB, have {w.config.stage_mb} MiB "
                         "(raise TCCL_STAGE_MB)")
    outs = {}
    grid = _gemm_ctas(w, pair)
    meta = 0
    if pair:
        meta = K["TCCL_RS_SYNC_ENTRY"] if _stage_handoff(w, "gemm_rs_pair") else 0
    else:
        _stage_handoff(w, "gemm_rs")
    Os = _locals(w, out) if out is not None else None
    arr = (L.GemmRsArgs * len(w.local_ranks))()
    for i, r in enumerate(w.local_ranks):
        ar, br = As[r], Bs[r]
        if ar.stride(1) != 1 or br.stride(1) != 1:
            raise ValueError("operands must have a unit inner stride")
        o = Os[r] if Os is not None else torch.empty((M // W, N), dtype=torch.bfloat16, device=ar.device)
        outs[r] = o
        arr[i] = L.GemmRsArgs(ar.data_ptr(), br.data_ptr(), o.data_ptr(), M, N, Kr, ar.stride(0), br.stride(0),
                              o.stride(0), _trace_ptr(w, trace, r, grid))
    stream = torch.cuda.current_stream(a0.device).cuda_stream
    fn = lib.tccl_gemm_reduce_scatter_pair if pair else lib.tccl_gemm_reduce_scatter
    if w.plans is not None:
        l = L.Launch(grid, 256, 0, meta, C.c_void_p(stream))
        rc = fn(C.byref(w.comm), C.byref(arr[0]), None, C.c_uint64(stage_bytes), C.byref(l))
    else:
        pb = int(lib.tccl_gemm_rs_pair_param_bytes() if pair else lib.tccl_gemm_rs_param_bytes())
        scratch = torch.empty(pb * W + 64, dtype=torch.uint8, device=a0.device)
        base = (scratch.data_ptr() + 63) & ~63
        w._keep.append(scratch)
        l = L.Launch(grid, 256, W, meta, C.c_void_p(stream))
        rc = fn(C.c_void_p(w.comms_dev.data_ptr()), arr, C.c_void_p(base), C.c_uint64(stage_bytes), C.byref(l))
    L.check(rc, "tccl_gemm_reduce_scatter_pair" if pair else "tccl_gemm_reduce_scatter")
    w.launches += 1
    if out is not None:
        return out
    return [outs[r] for r in w.local_ranks] if w.plans is None else outs[w.local_ranks[0]]


def ag_pair_schedule(W: int, rank: int, tm: int, tn: int, pairs: int, nbatch: int, k: int, *, halves: bool = True,
                     ring: bool = False, pair_tflops: float = 20.0, link_gbs: float = 600.0, start_us: float = 8.0,
                     round_us: float = 2.0):
    """Plan of the all-gather -> GEMM pair kernel: for every CTA pair the tiles it runs, in order.

    The kernel's built-in order deals tile ``pair + i * pairs`` to a pair whatever the moment its rows
    arrive; at 8 ranks most pairs then sit on a remote tile while others queue two tiles behind theirs.
    This is list scheduling against a small cost model instead: the rank's own rows are there at once,
    batch ``b`` of the peers' rows (``nbatch`` batches of ``tm / nbatch`` 128-row tiles per rank) after
    ``start_us + (b + 1) / nbatch`` of the time the link needs for all of them (``ring``: the movers send
    destination by destination, so the rows of rank ``rank - j`` are there after ``j`` rounds of one shard
    each plus ``round_us`` per round), a 256 x 256 tile costs ``2 * 256 * 256 * k / pair_tflops``.  Tiles are taken in the order their rows arrive and handed to
    the pair that is free first; the last tiles (those of the last batch, one wave at most) are cut into
    256 x 128 halves so that the work left when the last rows land spreads over all pairs.  Returns
    ``pairs`` lists of ``(mt, nt, half)`` (``mt`` = even 128-row tile index, ``half`` 0 / 1 / 2 = whole
    tile / left / right half).  Any plan that names every tile once is correct — the kernel waits for
    the rows of whatever tile it is given — the model only decides how good it is."""
    import heapq

    tm2 = tm // 2
    rows_in = (W - 1) * tm * 128
    link_us = rows_in * k * 2 / (link_gbs * 1e3)
    arrive = [start_us + (b + 1) / nbatch * link_us for b in range(nbatch)]
    tile_us = 2.0 * 256 * 256 * k / (pair_tflops * 1e6)
    units = []  # (ready, mt, nt, group): group = batch (or round) the rows come with, -1 = own
    for rt2 in range(tm2):
        for nt in range(tn):
            units.append((0.0, rank * tm + 2 * rt2, nt, -1))
    last = nbatch - 1
    if ring:
        shard_us = tm * 128 * k * 2 / (link_gbs * 1e3)
        last = W - 1
        for j in range(1, W):
            src = (rank - j) % W
            for rt2 in range(tm2):
                for nt in range(tn):
                    units.append((start_us + j * (shard_us + round_us), src * tm + 2 * rt2, nt, j))
    else:
        for rt2 in range(tm2):
            b = min(nbatch - 1, (2 * rt2 + 1) * nbatch // tm)
            for j in range(1, W):
                src = (rank + j) % W
                for nt in range(tn):
                    units.append((arrive[b], src * tm + 2 * rt2, nt, b))
    units.sort(key=lambda u: u[0])  # stable: own rows, then batch by batch
    n_last = sum(1 for u in units if u[3] == last)
    split_from = len(units) - min(n_last, pairs) if (halves and W > 1) else len(units)
    free = [(0.0, p) for p in range(pairs)]
    heapq.heapify(free)
    plan = [[] for _ in range(pairs)]
    for idx, (ready, mt, nt, _) in enumerate(units):
        parts = ((0, tile_us),) if idx < split_from else ((1, tile_us / 2 + 1.0), (2, tile_us / 2 + 1.0))
        for half, dur in parts:
            t, p = heapq.heappop(free)
            plan[p].append((mt, nt, half))
            heapq.heappush(free, (max(t, ready) + dur, p))
    return plan


def _ag_sched_tensor(w, r: int, tm: int, tn: int, pairs: int, nbatch: int, k: int, halves: bool, device):
    cache = w.__dict__.setdefault("_ag_sched", {})
    cfg = w.config
    key = (r, tm, tn, pairs, nbatch, k, halves, bool(cfg.ag_ring), cfg.ag_pair_tflops, cfg.ag_link_gbs)
    t = cache.get(key)
    if t is None:
        plan = ag_pair_schedule(w.world_size, r, tm, tn, pairs, nbatch, k, halves=halves, ring=bool(cfg.ag_ring),
                                pair_tflops=cfg.ag_pair_tflops, link_gbs=cfg.ag_link_gbs)
        stride = max(len(x) for x in plan) + 1
        rows = [[m | (n << 12) | (h << 28) for (m, n, h) in x] + [-1] * (stride - len(x)) for x in plan]
        t = cache[key] = torch.tensor(rows, dtype=torch.int32).to(device)
    return t


def all_gather_gemm(a_shard, bt, a_full=None, out=None, *, comm_ctas: int = 0, swiglu: bool = False, trace=None,
                    lsu_movers: bool = False, variant: str = "auto", world: Optional[WorldBase] = None):
    """``out_r = all_gather(a_shard) @ bt_r.T`` — tensor-parallel up-projection
    fused with the all-gather of the token rows.

    ``a_shard``: this rank's ``[M / W, K]`` rows (bf16, any device memory), ``bt``:
    its ``[N_r, K]`` weight slice.  ``a_full`` is the ``[M, K]`` gathered buffer in
    symmetric memory (allocated and cached per shape when omitted); it holds the
    gathered activations afterwards.  Returns ``(out, a_full)`` with ``out`` the
    rank's ``[M, N_r]`` result.  ``M % (128 W) == 0``.

    ``swiglu=True`` fuses the gated activation into the epilogue: ``bt`` must be
    packed by :func:`pack_gate_up` (every 256-row block = 128 gate rows, then the
    128 matching up rows) and ``out`` is ``[M, N_r / 2] = silu(gate) * up``.

    ``variant``: ``"pair"`` = 256 x 256 tiles on pairs of SMs, every CTA moves its share of the
    shard before it computes (needs ``M % (256 W) == 0``); ``"single"`` = 128 x 256 single-CTA
    tiles with ``comm_ctas`` dedicated data movers; ``"auto"`` = pair when the shape allows.  When
    the pair kernel allocates the gathered buffer itself it keeps two of them and alternates (so it
    needs no barrier on entry): the returned ``a_full`` is the one this call filled, and it stays
    valid until the call after the next one."""
    w = get_world(world)
    W = w.world_size
    As, Bs = _locals(w, a_shard), _locals(w, bt)
    a0, b0 = As[w.local_ranks[0]], Bs[w.local_ranks[0]]
    if a0.dtype != torch.bfloat16 or b0.dtype != torch.bfloat16:
        raise TypeError("all_gather_gemm takes bfloat16 operands")
    rows, Kd = a0.shape
    M, N = rows * W, b0.shape[0]
    if b0.shape[1] != Kd:
        raise ValueError("a_shard is [M / W, K], bt is [N, K]")
    if rows % 128 or N % 8 or Kd % 8:
        raise ValueError(f"need (M / W) % 128 == 0, N % 8 == 0, K % 8 == 0 (got M/W={rows}, N={N}, K={Kd})")
    if swiglu and N % 256:
        raise ValueError("swiglu needs N % 256 == 0 (whole gate|up tiles)")
    n_out = N // 2 if swiglu else N
    if variant not in ("auto", "pair", "single"):
        raise ValueError("variant must be 'auto', 'pair' or 'single'")
    pair_ok = rows % 256 == 0
    if variant == "pair" and not pair_ok:
        raise ValueError("the pair kernel needs (M / W) % 256 == 0")
    pair = pair_ok and variant != "single"
    half_bytes = 0
    ret_full = a_full
    seq = 0
    if pair:  # mirrors the device's count of pair calls, which picks the half (see reset())
        seq = w.__dict__.get("_ag_seq", 0)
        w.__dict__["_ag_seq"] = seq + 1
    if a_full is None:
        cache = w.__dict__.setdefault("_ag_buffers", {})
        key = (M, Kd, pair)
        a_full = cache.get(key)
        if a_full is None:
            a_full = cache[key] = w.empty((2, M, Kd) if pair else (M, Kd), torch.bfloat16)
        ret_full = a_full
        if pair:
            half_bytes = M * Kd * 2
            if w.plans is not None:
                ret_full = a_full[seq & 1]
            else:
                from ..parallel.emu import EmuTensor
                ret_full = EmuTensor([t[seq & 1] for t in a_full.parts])
    full_ptrs = w.peer_ptrs(a_full)
    # two ranks: the switch would deliver every row to its sender too (twice the inbound bytes of a plain store)
    mc = w.mc_ptr(a_full) if ((W > 2 and not w.config.ag_ring) or not pair) else 0
    lib = L.lib()
    lib.tccl_ag_gemm_param_bytes.restype = C.c_uint64
    lib.tccl_ag_gemm_pair_param_bytes.restype = C.c_uint64
    grid = _gemm_ctas(w, pair)
    if comm_ctas <= 0:
        # Few data movers: every mover CTA is an SM the GEMM does not get, and 8 movers
        # with 8 vectors per thread in flight already fill the link (measured on 8xB200,
        # Llama-3-8B up-projection: 8 movers 116 us, 16: 121 us, 24: 125 us, 48: 128 us).
        comm_ctas = w.config.ag_movers if grid > 16 else 2
        comm_ctas = max(1, min(comm_ctas, grid - 1))
    outs = {}
    Os = _locals(w, out) if out is not None else None
    arr = (L.AgGemmArgs * len(w.local_ranks))()
    for i, r in enumerate(w.local_ranks):
        ar, br = As[r], Bs[r]
        if ar.stride(1) != 1 or br.stride(1) != 1:
            raise ValueError("operands must have a unit inner stride")
        o = Os[r] if Os is not None else torch.empty((M, n_out), dtype=torch.bfloat16, device=ar.device)
        if o.shape != (M, n_out) or o.dtype != torch.bfloat16 or o.stride(1) != 1:
            raise ValueError(f"out must be bf16 [{M}, {n_out}] with a unit inner stride")
        outs[r] = o
        g = L.AgGemmArgs()
        g.a_shard = ar.data_ptr()
        for q, v in enumerate(full_ptrs):
            g.a_full[q] = v
        g.mc_a_full = mc
        g.bt, g.out = br.data_ptr(), o.data_ptr()
        g.m, g.n, g.k = M, N, Kd
        g.lda_shard, g.lda_full, g.ldb, g.ldo = ar.stride(0), Kd, br.stride(0), o.stride(0)
        g.comm_ctas = max(1, int(w.config.ag_batches)) if pair else comm_ctas  # pair kernel: batches of the mover phase
        g.swiglu = 1 if swiglu else 0
        g.trace = _trace_ptr(w, trace, r, grid)
        g.lsu_movers = int(lsu_movers)
        if pair:  # bits: 2 = move the shard only (timeline tool), 4 = movers send destination by destination
            g.lsu_movers = (2 if int(lsu_movers) == 2 else 0) | (4 if w.config.ag_ring else 0)
        if pair and w.config.ag_schedule and W > 1:
            nb = max(1, min(int(w.config.ag_batches), rows // 128))
            sched = _ag_sched_tensor(w, r, rows // 128, -(-N // 256), grid // 2, nb, Kd, True, ar.device)
            g.sched, g.sched_stride = sched.data_ptr(), sched.shape[1]
        arr[i] = g
    stream = torch.cuda.current_stream(a0.device).cuda_stream
    if pair:
        fn = lib.tccl_allgather_gemm_pair
        extra = (C.c_uint64(half_bytes),)
    else:
        fn = lib.tccl_allgather_gemm
        extra = ()
    if w.plans is not None:
        l = L.Launch(grid, 256, 0, 0, C.c_void_p(stream))
        rc = fn(C.byref(w.comm), C.byref(arr[0]), None, *extra, C.byref(l))
    else:
        pb = int(lib.tccl_ag_gemm_pair_param_bytes() if pair else lib.tccl_ag_gemm_param_bytes())
        scratch = torch.empty(pb * W + 64, dtype=torch.uint8, device=a0.device)
        base = (scratch.data_ptr() + 63) & ~63
        w._keep.append(scratch)
        l = L.Launch(grid, 256, W, 0, C.c_void_p(stream))
        rc = fn(C.c_void_p(w.comms_dev.data_ptr()), arr, C.c_void_p(base), *extra, C.byref(l))
    L.check(rc, "tccl_allgather_gemm_pair" if pair else "tccl_allgather_gemm")
    w.launches += 1
    res = out if out is not None else ([outs[r] for r in w.local_ranks] if w.plans is None else outs[w.local_ranks[0]])
    return res, ret_full


def all_reduce_bias_residual_rmsnorm(x, weight, bias=None, residual=None, eps: float = 1e-5, out=None,
                                     residual_out=None, *, algo: str = "auto", world: Optional[WorldBase] = None):
    """``y = RMSNorm(all_reduce(x) + bias + residual) * weight`` in one kernel.

    ``x``: this rank's partial ``[tokens, hidden]`` in symmetric memory (the output
    of a row-parallel linear before its reduction).  ``bias`` / ``weight``:
    ``[hidden]``; ``residual``: this rank's (replicated) ``[tokens, hidden]``.
    ``out`` (and ``residual_out``, the pre-norm sum that becomes the next residual)
    live in symmetric memory because every rank writes its rows into all of them;
    they are allocated and cached per shape when omitted (pass ``residual_out=True``
    to ask for the pre-norm sum).  Returns ``y`` or ``(y, residual_out)``."""
    w = get_world(world)
    check_sym_tensor(w, x, "input")
    x0 = w.local(x, w.local_ranks[0])
    if x0.dim() != 2:
        raise ValueError("x must be [tokens, hidden]")
    T, H = x0.shape
    dt = dtype_code(x0.dtype)
    vpt = 16 // x0.element_size()
    if H % vpt or H > 512 * 4 * vpt:
        raise ValueError(f"hidden must be a multiple of {vpt} and at most {512 * 4 * vpt}")
    cache = w.__dict__.setdefault("_arn_buffers", {})

    def sym(tag, given):
        if given is not None and given is not True:
            check_sym_tensor(w, given, tag)
            return given
        key = (tag, T, H, x0.dtype)
        if key not in cache:
            cache[key] = w.empty((T, H), x0.dtype)
        return cache[key]

    out = sym("out", out)
    want_res = residual_out is not None and residual_out is not False
    res_out = sym("residual_out", residual_out) if want_res else None
    if algo == "auto":
        algo = "nvls" if w.has_nvls and w.world_size > 2 else "p2p"
    if algo == "nvls" and not w.has_nvls:
        raise RuntimeError("nvls variant needs NVLS multicast")
    Ws, Bs, Rs = _locals(w, weight), (_locals(w, bias) if bias is not None else None), \
        (_locals(w, residual) if residual is not None else None)
    xp, op = w.peer_ptrs(x), w.peer_ptrs(out)
    rp = w.peer_ptrs(res_out) if want_res else None
    args = {}
    for r in w.local_ranks:
        a = L.ArnArgs()
        for q in range(w.world_size):
            a.x[q], a.out[q] = xp[q], op[q]
            a.res_out[q] = rp[q] if rp else 0
        a.mc_x, a.mc_out = w.mc_ptr(x), w.mc_ptr(out)
        a.mc_res_out = w.mc_ptr(res_out) if want_res else 0
        for name, src in (("weight", Ws), ("bias", Bs), ("residual", Rs)):
            if src is None:
                setattr(a, name, 0)
                continue
            tns = src[r]
            if tns.dtype != x0.dtype or not tns.is_contiguous() or tns.data_ptr() % 16:
                raise ValueError(f"{name} must be contiguous, 16-byte aligned and of x's dtype")
            if tns.numel() != (T * H if name == "residual" else H):
                raise ValueError(f"{name} has the wrong size")
            setattr(a, name, tns.data_ptr())
        a.eps, a.tokens, a.hidden, a.dtype = float(eps), T, H, dt
        a.flags = w.coll_flags()
        args[r] = a
    rows = -(-T // w.world_size)
    nv = H // vpt
    per_sm = 2 if nv <= 512 and w.plans is not None else 1  # narrow rows: two CTAs per SM
    batch = 1                                                # rows a CTA handles together (kernel's R)
    grid = max(1, min(-(-rows // batch), w.max_ctas() * per_sm, K["TCCL_MAX_BLOCKS"]))
    fn = L.lib().tccl_allreduce_bias_residual_rmsnorm
    nvls = 1 if algo == "nvls" else 0
    stream = torch.cuda.current_stream(x0.device).cuda_stream
    if w.plans is not None:
        l = L.Launch(grid, 512, 0, dt, C.c_void_p(stream))
        rc = fn(C.byref(w.comm), C.byref(args[w.local_ranks[0]]), nvls, H, C.byref(l))
    else:
        arr = (L.ArnArgs * w.world_size)(*[args[r] for r in w.local_ranks])
        dev = w._to_device(arr)
        w._keep.append(dev)
        l = L.Launch(grid, 512, w.world_size, dt, C.c_void_p(stream))
        rc = fn(C.c_void_p(w.comms_dev.data_ptr()), C.c_void_p(dev.data_ptr()), nvls, H, C.byref(l))
    L.check(rc, "tccl_allreduce_bias_residual_rmsnorm")
    w.launches += 1
    return (out, res_out) if want_res else out


def pack_gate_up(gate_w: torch.Tensor, up_w: torch.Tensor) -> torch.Tensor:
    """Interleave ``gate_w`` and ``up_w`` (both ``[F, K]``, ``F % 128 == 0``) in
    blocks of 128 rows — gate rows ``[128 j, 128 j + 128)`` followed by the same
    rows of ``up_w`` — which is the weight layout the ``swiglu`` epilogue of
    :func:`all_gather_gemm` expects (one 256-wide output tile = 128 gate columns
    and the 128 up columns they multiply)."""
    F, Kd = gate_w.shape
    if up_w.shape != gate_w.shape or F % 128:
        raise ValueError("gate and up weights must both be [F, K] with F % 128 == 0")
    return torch.stack([gate_w.view(F // 128, 128, Kd), up_w.view(F // 128, 128, Kd)], dim=1).reshape(2 * F, Kd).contiguous()
