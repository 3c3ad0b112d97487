"""Flat collectives and barriers with all ranks emulated on one GPU, against a
plain PyTorch fp32 reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.bfloat16, torch.float32, torch.float16]
TOL = {torch.bfloat16: 2 ** -8, torch.float16: 2 ** -11, torch.float32: 1e-6}


def make_inputs(world, W, n, dtype, seed):
    parts = []
    for r in range(W):
        g = torch.Generator(device="cpu").manual_seed(seed + r)
        parts.append(torch.randn(n, generator=g, dtype=torch.float32).to(dtype))
    return world.from_parts(parts)


def ref_sum(x):
    return torch.stack([p.float() for p in x.parts]).sum(0)


def assert_close_to_sum(out, ref, dtype, W):
    # one rounding of an fp32 sum: half an ulp of the result, relative
    err = (out.float() - ref).abs()
    bound = ref.abs() * TOL[dtype] + 1e-6 * W
    assert bool((err <= bound).all()), f"max err {err.max().item()} (bound {bound.max().item()})"


@pytest.mark.parametrize("W", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("rounds,blocks", [(1, 1), (3, 7), (50, 16)])
def test_barrier_p2p(emu_worlds, W, rounds, blocks):
    import tccl_b200 as tccl

    from tccl_b200.utils.lib import K

    w = emu_worlds(W)
    epochs = lambda r: w.local_states[r][K["TCCL_LOCAL_EPOCH"] : K["TCCL_LOCAL_EPOCH"] + blocks].clone()
    before = [epochs(r) for r in range(W)]
    tccl.barrier(world=w, blocks=blocks, threads=64, rounds=rounds)
    tccl.barrier(world=w, blocks=blocks, threads=64, rounds=rounds)
    torch.cuda.synchronize()
    w.check()
    for r in range(W):
        assert bool((epochs(r) - before[r] == 2 * rounds).all())


@pytest.mark.parametrize("W", [1, 2, 4, 8])
def test_barrier_cas_on_pads_resets_to_zero(emu_worlds, W):
    import tccl_b200 as tccl
    from tccl_b200.parallel.emu import EmuTensor

    w = emu_worlds(W)
    pads = EmuTensor([torch.zeros(32 * W, dtype=torch.int32, device=w.device) for _ in range(W)])
    for _ in range(5):
        tccl.barrier_test(world=w, pads=pads, blocks=16 if W == 8 else 32, threads=128)
    torch.cuda.synchronize()
    w.check()
    for p in pads:
        assert int(p.abs().sum()) == 0


@pytest.mark.parametrize("W", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [8, 4096 + 8, 100003, 1 << 20])
def test_all_reduce_oneshot(emu_worlds, W, dtype, n):
    import tccl_b200 as tccl

    w = emu_worlds(W)
    x = make_inputs(w, W, n, dtype, 1000)
    keep = [p.clone() for p in x.parts]
    out = tccl.all_reduce(x, algo="oneshot_p2p", world=w)
    torch.cuda.synchronize()
    w.check()
    ref = ref_sum(x)
    for r in range(W):
        assert_close_to_sum(out[r], ref, dtype, W)
        assert torch.equal(out[r], out[0])
        assert torch.equal(x[r], keep[r])


def test_all_reduce_fill_rank_exact(emu_worlds):
    """The reference's own check: fill with the rank, expect W (W-1) / 2
    (triton_one_shot_all_reduce_no_128.py:116-127)."""
    import tccl_b200 as tccl

    W = 8
    w = emu_worlds(W)
    x = w.from_parts([torch.full((8192,), float(r), dtype=torch.bfloat16) for r in range(W)])
    out = tccl.one_shot_all_reduce(x, world=w)
    torch.cuda.synchronize()
    for r in range(W):
        assert bool(out[r].eq(W * (W - 1) // 2).all())


@pytest.mark.parametrize("W", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", [8, 1000, 65536 + 24, 3 * (1 << 20) + 5])
def test_all_reduce_twoshot_inplace(emu_worlds, W, dtype, n):
    import tccl_b200 as tccl

    w = emu_worlds(W)
    x = make_inputs(w, W, n, dtype, 2000)
    ref = ref_sum(x)
    res = tccl.all_reduce(x, inplace=True, algo="twoshot_p2p", world=w)
    torch.cuda.synchronize()
    w.check()
    assert res is x
    for r in range(W):
        assert_close_to_sum(x[r], ref, dtype, W)
        assert torch.equal(x[r], x[0])


@pytest.mark.parametrize("W", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(8, 4, 4), (4, 8, 8), (12, 3, 2)])  # (reducer warps, stages, unroll)
@pytest.mark.parametrize("n", [8, 65536 + 24, 3 * (1 << 20) + 5])
def test_all_reduce_twoshot_pipelined(emu_worlds, W, dtype, shape, n):
    """Reducer and broadcaster warps decoupled through a shared-memory ring: in place, twice in a
    row (the second call finds the mbarriers re-initialised), for several shapes of the pipeline."""
    import tccl_b200 as tccl

    w = emu_worlds(W)
    old = (w.config.pipe_reducers, w.config.pipe_stages, w.config.pipe_unroll)
    w.config.pipe_reducers, w.config.pipe_stages, w.config.pipe_unroll = shape
    try:
        for seed in (2000, 2100):
            x = make_inputs(w, W, n, dtype, seed)
            ref = ref_sum(x)
            res = tccl.all_reduce(x, inplace=True, algo="twoshot_pipe_p2p", world=w)
            torch.cuda.synchronize()
            w.check()
            assert res is x
            for r in range(W):
                assert_close_to_sum(x[r], ref, dtype, W)
                assert torch.equal(x[r], x[0])
    finally:
        w.config.pipe_reducers, w.config.pipe_stages, w.config.pipe_unroll = old


@pytest.mark.parametrize("W", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", [8, 1000, 65536 + 24, 3 * (1 << 20) + 5, 12 * (1 << 20)])
def test_all_reduce_twoshot_bulk_copies(emu_worlds, W, dtype, n):
    """The two-shot kernel that moves its data with bulk async copies (loader / reducers / storer around
    shared-memory stages): in place twice in a row, then into a separate symmetric tensor."""
    import tccl_b200 as tccl

    w = emu_worlds(W)
    for seed in (2000, 2100):
        x = make_inputs(w, W, n, dtype, seed)
        ref = ref_sum(x)
        res = tccl.all_reduce(x, inplace=True, algo="twoshot_bulk_p2p", world=w)
        torch.cuda.synchronize()
        w.check()
        assert res is x
        for r in range(W):
            assert_close_to_sum(x[r], ref, dtype, W)
            assert torch.equal(x[r], x[0])
    x = make_inputs(w, W, n, dtype, 2200)
    keep = [p.clone() for p in x.parts]
    ref = ref_sum(x)
    out = w.empty(n, dtype)
    tccl.all_reduce(x, out=out, algo="twoshot_bulk_p2p", world=w)
    torch.cuda.synchronize()
    w.check()
    for r in range(W):
        assert torch.equal(x[r], keep[r])
        assert_close_to_sum(out[r], ref, dtype, W)


def test_all_reduce_twoshot_symmetric_out_keeps_input(emu_worlds):
    import tccl_b200 as tccl

    W, n = 4, 50000
    w = emu_worlds(W)
    x = make_inputs(w, W, n, torch.bfloat16, 7)
    keep = [p.clone() for p in x.parts]
    out = w.empty(n, torch.bfloat16)
    tccl.all_reduce(x, out=out, algo="twoshot_p2p", world=w)
    torch.cuda.synchronize()
    ref = ref_sum(x)
    for r in range(W):
        assert torch.equal(x[r], keep[r])
        assert_close_to_sum(out[r], ref, torch.bfloat16, W)


def test_auto_choice_and_views(emu_worlds):
    """Views with a storage offset (tensor[:size], as every reference bench uses)."""
    import tccl_b200 as tccl

    W = 4
    w = emu_worlds(W)
    big = make_inputs(w, W, 1 << 16, torch.bfloat16, 11)
    for lo, hi in [(0, 4096), (8, 8 + 1024), (1 << 15, 1 << 16)]:
        v = big[lo:hi]
        out = tccl.all_reduce(v, world=w)
        torch.cuda.synchronize()
        ref = ref_sum(v)
        for r in range(W):
            assert_close_to_sum(out[r], ref, torch.bfloat16, W)
    with pytest.raises(ValueError):
        tccl.all_reduce(big[3:11], world=w)  # 6-byte offset: not 16-byte aligned


@pytest.mark.parametrize("W", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [8, 1003, 1 << 18])
def test_all_gather_pull(emu_worlds, W, dtype, n):
    import tccl_b200 as tccl

    w = emu_worlds(W)
    parts = []
    for r in range(W):
        g = torch.Generator(device="cpu").manual_seed(3000 + r)
        parts.append((torch.rand(n, generator=g) * 2 - 1).to(dtype))
    x = w.from_parts(parts)
    out = tccl.one_shot_all_gather(x, W, world=w)
    torch.cuda.synchronize()
    w.check()
    ref = torch.stack(list(x.parts))
    for r in range(W):
        assert out[r].shape == (W, n)
        assert torch.equal(out[r], ref)


@pytest.mark.parametrize("W", [2, 4, 8])
@pytest.mark.parametrize("n", [8, 1 << 12, (1 << 16) + 8])
def test_all_gather_push(emu_worlds, W, n):
    import tccl_b200 as tccl

    w = emu_worlds(W)
    x = make_inputs(w, W, n, torch.bfloat16, 3000)
    out = w.empty((W, n), torch.bfloat16)
    tccl.all_gather(x, out=out, algo="push", world=w)
    torch.cuda.synchronize()
    w.check()
    ref = torch.stack(list(x.parts))
    for r in range(W):
        assert torch.equal(out[r], ref)


@pytest.mark.parametrize("W", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("per_vec", [1, 37, 4096])
def test_reduce_scatter(emu_worlds, W, dtype, per_vec):
    import tccl_b200 as tccl

    vpt = 16 // torch.empty(0, dtype=dtype).element_size()
    n = per_vec * vpt * W
    w = emu_worlds(W)
    x = make_inputs(w, W, n, dtype, 3000)
    out = tccl.one_shot_reduce_scatter(x, world=w)
    torch.cuda.synchronize()
    w.check()
    ref = ref_sum(x).view(W, -1)
    for r in range(W):
        assert_close_to_sum(out[r], ref[r], dtype, W)
    with pytest.raises(ValueError):
        tccl.reduce_scatter(x[: n - vpt] if W > 1 else x[:1], world=w)


def test_back_to_back_stress_changing_data(emu_worlds):
    """1000 calls with the inputs rewritten between calls: a missing exit barrier
    (write-after-read) or entry barrier (read-before-write) shows up as a wrong sum."""
    import tccl_b200 as tccl

    W, n = 4, 2048
    w = emu_worlds(W)
    x = w.empty(n, torch.float32)
    for it in range(1000):
        for r in range(W):
            x[r].fill_(float(it * (r + 1)))
        o = tccl.all_reduce(x, algo="oneshot_p2p", world=w)
        if it % 100 == 99:
            torch.cuda.synchronize()
            expect = float(it * sum(range(1, W + 1)))
            assert bool((o[0] == expect).all()) and bool((o[W - 1] == expect).all())
    w.check()


def test_timeout_is_reported_not_hung(emu_worlds):
    """A wait that nothing satisfies returns after the limit with a TIMEOUT
    status; the context stays usable and reset() clears the state."""
    import time

    import tccl_b200 as tccl
    from tccl_b200.utils.lib import TcclTimeout

    w = emu_worlds(2)
    w.set_timeout_ms(200.0)
    try:
        t0 = time.time()
        tccl.wait_never(world=w)
        torch.cuda.synchronize()
        assert time.time() - t0 < 5.0
        st = w.last_status(0)
        assert st["code"] == 1 and st["where"] == "TCCL_W_SIGNAL" and st["aborted"]
        with pytest.raises(TcclTimeout):
            w.check()
    finally:
        w.reset()
        w.set_timeout_ms(2000.0)
    w.check()
    x = make_inputs(w, 2, 1024, torch.bfloat16, 5)
    out = tccl.all_reduce(x, world=w)
    torch.cuda.synchronize()
    assert_close_to_sum(out[0], ref_sum(x), torch.bfloat16, 2)


@pytest.mark.parametrize("W", [1, 2, 3, 4, 5, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n,chunk_kb,ll", [(8, 512, False), (8, 512, True), (4096, 1, False), (4096, 1, True),
                                           (100000, 4, False), (65536 + 24, 4, True), ((1 << 20) + 64, 64, False),
                                           (3 << 20, 512, False)])
def test_double_tree_all_reduce(emu_worlds, W, dtype, n, chunk_kb, ll):
    """`ll`: small messages take the kernel whose lines carry their own flags; with it switched off
    the same sizes exercise the chunked kernel (ring, counters, acknowledgements) with tiny chunks."""
    import tccl_b200 as tccl

    w = emu_worlds(W)
    old = w.config.tree_chunk_bytes
    old_ll = w.config.tree_ll_max_bytes
    w.config.tree_chunk_bytes = chunk_kb * 1024
    w.config.tree_ll_max_bytes = old_ll if ll else 0
    try:
        x = make_inputs(w, W, n, dtype, 2000)
        keep = [p.clone() for p in x.parts]
        ref = ref_sum(x)
        out = tccl.double_tree_all_reduce(x, world=w)
        torch.cuda.synchronize()
        w.check()
        for r in range(W):
            # tree order != rank order: a few roundings of partial sums on the way up
            err = (out[r].float() - ref).abs()
            steps = max(1, W.bit_length())
            assert bool((err <= ref.abs() * TOL[dtype] * steps + (2e-2 if dtype != torch.float32 else 1e-5) * steps).all())
            assert torch.equal(out[r], out[0])
            assert torch.equal(x[r], keep[r])
        # a second out-of-place call hands back a new tensor, not the first one's storage
        out_b = tccl.double_tree_all_reduce(x, world=w)
        torch.cuda.synchronize()
        for r in range(W):
            assert out_b[r].data_ptr() != out[r].data_ptr() and torch.equal(out_b[r], out[r])
        # in place, twice in a row (the counters are running totals: nothing is reset in between)
        for _ in range(2):
            y = w.from_parts([p.clone() for p in keep])
            tccl.all_reduce(y, inplace=True, algo="tree", world=w)
            torch.cuda.synchronize()
            w.check()
            for r in range(W):
                assert torch.equal(y[r], out[0])
    finally:
        w.config.tree_chunk_bytes = old
        w.config.tree_ll_max_bytes = old_ll


@pytest.mark.parametrize("W", [1, 2, 3, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", [4096 + 8, (1 << 20) + 64, 3 << 20])
def test_double_tree_push_and_pull_down_agree(emu_worlds, W, dtype, n):
    """The two forms of the way down (parents store into their children / children load from their
    parent and acknowledge) give the same bits, out of place and in place, twice in a row."""
    import tccl_b200 as tccl

    w = emu_worlds(W)
    old = (w.config.tree_pull_min_bytes, w.config.tree_ll_max_bytes)
    try:
        x = make_inputs(w, W, n, dtype, 2500)
        keep = [p.clone() for p in x.parts]
        w.config.tree_ll_max_bytes = 0
        w.config.tree_pull_min_bytes = 1 << 40
        push = tccl.double_tree_all_reduce(x, world=w)
        w.config.tree_pull_min_bytes = 0
        pull = tccl.double_tree_all_reduce(x, world=w)
        ys = []
        for _ in range(2):
            y = w.from_parts([p.clone() for p in keep])
            tccl.all_reduce(y, inplace=True, algo="tree", world=w)
            ys.append(y)
        torch.cuda.synchronize()
        w.check()
        for r in range(W):
            assert torch.equal(pull[r], push[r]) and torch.equal(x[r], keep[r])
            assert torch.equal(ys[0][r], push[r]) and torch.equal(ys[1][r], push[r])
    finally:
        w.config.tree_pull_min_bytes, w.config.tree_ll_max_bytes = old


@pytest.mark.parametrize("W", [2, 4, 8])
def test_double_tree_back_to_back_calls_of_changing_size(emu_worlds, W):
    """No barrier separates two tree all-reduces: sizes, chunking and CTA counts change from call
    to call while the ring and its counters carry on."""
    import tccl_b200 as tccl

    w = emu_worlds(W)
    old = w.config.tree_chunk_bytes
    sizes = [(1 << 16, 4096), (4096, 1024), ((1 << 18) + 8, 1 << 22), (8, 1 << 22), (1 << 16, 256)]
    try:
        pending = []
        for it in range(15):
            n, chunk = sizes[it % len(sizes)]
            w.config.tree_chunk_bytes = chunk
            x = make_inputs(w, W, n, torch.float32, 3000 + 16 * it)
            pending.append((tccl.double_tree_all_reduce(x, world=w), ref_sum(x)))
        torch.cuda.synchronize()
        w.check()
        for out, ref in pending:
            for r in range(W):
                assert bool(((out[r].float() - ref).abs() <= ref.abs() * 1e-5 + 1e-5).all())
    finally:
        w.config.tree_chunk_bytes = old


@pytest.mark.parametrize("W", [2, 3, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", [8, 512, 4096 + 8, 32768])
def test_all_reduce_push_small_messages(emu_worlds, W, dtype, n):
    """Push variant: the input is ordinary device memory; many calls in a row
    exercise the alternating slot parity without an exit barrier."""
    import tccl_b200 as tccl

    w = emu_worlds(W)
    for it in range(6):
        x = make_inputs(w, W, n, dtype, 7000 + 10 * it)
        ref = ref_sum(x)
        out = tccl.all_reduce(x, algo="push_p2p", world=w)
        torch.cuda.synchronize()
        w.check()
        for r in range(W):
            assert_close_to_sum(out[r], ref, dtype, W)
            assert torch.equal(out[r], out[0])
    # auto picks it for small messages, in place too
    y = make_inputs(w, W, n, dtype, 1)
    ref = ref_sum(y)
    tccl.all_reduce(y, inplace=True, world=w)
    torch.cuda.synchronize()
    for r in range(W):
        assert_close_to_sum(y[r], ref, dtype, W)


@pytest.mark.parametrize("W", [2, 4, 8])
def test_push_all_reduce_calls_of_alternating_size_and_grid(emu_worlds, W):
    """64 KiB, 32 KiB and 1 KiB pushes in turn, 1000 calls with changing data and no host
    synchronisation in between: the slot layout and the half in use must not depend on the
    message size or on the grid, or a later call lands in bytes an earlier one still sums."""
    import tccl_b200 as tccl

    w = emu_worlds(W)
    sizes = [16384, 8192, 256]  # fp32 elements
    data = {n: w.from_parts([torch.zeros(n) for _ in range(W)]) for n in sizes}
    checks = []
    for it in range(1000):
        n = sizes[it % 3]
        x = data[n]
        for r in range(W):
            x[r].fill_(float((it % 97) * (r + 1)))
        out = tccl.all_reduce(x, algo="push_p2p", world=w)
        if it % 40 in (37, 38, 39):
            checks.append((out, float((it % 97) * W * (W + 1) // 2)))
    torch.cuda.synchronize()
    w.check()
    for out, want in checks:
        for r in range(W):
            assert bool((out[r] == want).all())


def test_large_all_reduce_into_ordinary_memory_uses_the_staged_two_shot(emu_worlds):
    import tccl_b200 as tccl

    W, n = 4, (1 << 20) + 8
    w = emu_worlds(W)
    x = make_inputs(w, W, n, torch.bfloat16, 99)
    keep = [p.clone() for p in x.parts]
    ref = ref_sum(x)
    before = w.launches
    out = tccl.all_reduce(x, world=w)          # fresh output
    out2 = [torch.empty(n, dtype=torch.bfloat16, device=w.device) for _ in range(W)]
    from tccl_b200.parallel.emu import EmuTensor
    tccl.all_reduce(x, out=EmuTensor(out2), world=w)
    torch.cuda.synchronize()
    w.check()
    assert w.launches == before + 2
    for r in range(W):
        assert_close_to_sum(out[r], ref, torch.bfloat16, W)
        assert torch.equal(out2[r], out[r]) and torch.equal(x[r], keep[r])
