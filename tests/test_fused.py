"""Fused compute + collective kernels with emulated ranks, against an fp32
single-GPU PyTorch reference of the same operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(shape, seed, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).cuda()


@pytest.mark.parametrize("variant", ["single", "pair"])
@pytest.mark.parametrize("W,M,N,K", [(1, 256, 256, 128), (2, 256, 256, 64), (2, 512, 512, 1792), (4, 1024, 512, 448),
                                     (8, 1024, 256, 224), (4, 2048, 1024, 1792), (8, 2048, 512, 224),
                                     (2, 1024, 768, 8), (3, 768, 256, 72)])
def test_gemm_reduce_scatter(emu_worlds, W, M, N, K, variant):
    import tccl_b200 as tccl

    if variant == "pair" and M % (256 * W):
        pytest.skip("the pair kernel needs whole 256-row tiles per rank")
    w = emu_worlds(W)
    a = [_rand((M, K), 4000 + r) for r in range(W)]
    bt = [_rand((N, K), 5000 + r, 0.02) for r in range(W)]
    for rep in range(3):  # several times: epochs advance together and the staging halves alternate
        outs = tccl.gemm_reduce_scatter(a, bt, variant=variant, world=w)
        torch.cuda.synchronize()
        w.check()
        ref = sum(a[r].float() @ bt[r].float().t() for r in range(W))
        rows = M // W
        for r in range(W):
            got = outs[r].float()
            exp = ref[r * rows:(r + 1) * rows]
            err = (got - exp).abs()
            # W-1 partials travel as bf16 (each rounded once), then one final rounding
            bound = exp.abs() * 2 ** -8 + 2 ** -8 * W * 0.02 * (K ** 0.5) * 3 + 1e-3
            assert bool((err <= bound).all()), f"rank {r}: max err {err.max().item()} ratio {(err / bound).max().item()}"


@pytest.mark.parametrize("variant", ["single", "pair"])
@pytest.mark.parametrize("W,M,N,K", [(1, 256, 256, 128), (2, 256, 512, 64), (2, 1024, 1792, 512), (4, 1024, 264, 448),
                                     (8, 1024, 256, 256), (4, 2048, 1792, 1024), (8, 2048, 264, 256), (3, 768, 520, 72)])
def test_all_gather_gemm(emu_worlds, W, M, N, K, variant):
    import tccl_b200 as tccl

    if variant == "pair" and M % (256 * W):
        pytest.skip("the pair kernel needs whole 256-row tiles per rank")
    w = emu_worlds(W)
    rows = M // W
    shards = [_rand((rows, K), 4000 + r) for r in range(W)]
    bt = [_rand((N, K), 5000 + r, 0.02) for r in range(W)]
    a_all = torch.cat(shards).float()
    for rep in range(3):
        outs, a_full = tccl.all_gather_gemm(shards, bt, variant=variant, world=w)
        torch.cuda.synchronize()
        w.check()
        for r in range(W):
            ref = a_all @ bt[r].float().t()
            err = (outs[r].float() - ref).abs()
            bound = ref.abs() * 2 ** -8 + 1e-3 * (K ** 0.5) * 0.02
            assert bool((err <= bound).all()), f"rank {r}: max err {err.max().item()} ratio {(err / bound).max().item()}"
            assert torch.equal(a_full[r].float(), a_all)  # the gathered activations are left behind, exactly


@pytest.mark.parametrize("planned", [True, False])
@pytest.mark.parametrize("batches", [0, 1, 3, 4, 64])
@pytest.mark.parametrize("W,M,N,K", [(2, 2048, 512, 256), (4, 2048, 264, 448), (8, 4096, 256, 128)])
def test_all_gather_gemm_pair_batch_counts(emu_worlds, W, M, N, K, batches, planned):
    """The mover phase may send the shard in any number of batches (capped at one per row tile), and the
    tiles may follow the host's plan (with half tiles at the end) or the kernel's built-in order."""
    import tccl_b200 as tccl

    w = emu_worlds(W)
    old = (w.config.ag_batches, w.config.ag_schedule, w.config.ag_ring)
    # batches == 0: the ring-ordered movers (destination by destination); else batches to all ranks at once
    w.config.ag_batches, w.config.ag_schedule, w.config.ag_ring = max(1, batches), planned, batches == 0
    try:
        shards = [_rand((M // W, K), 4100 + r) for r in range(W)]
        bt = [_rand((N, K), 5100 + r, 0.02) for r in range(W)]
        a_all = torch.cat(shards).float()
        for rep in range(2):
            outs, a_full = tccl.all_gather_gemm(shards, bt, variant="pair", world=w)
            torch.cuda.synchronize()
            w.check()
            for r in range(W):
                ref = a_all @ bt[r].float().t()
                err = (outs[r].float() - ref).abs()
                assert bool((err <= ref.abs() * 2 ** -8 + 1e-3 * (K ** 0.5) * 0.02).all())
                assert torch.equal(a_full[r].float(), a_all)
    finally:
        w.config.ag_batches, w.config.ag_schedule, w.config.ag_ring = old


@pytest.mark.parametrize("W", [1, 2, 4, 8])
@pytest.mark.parametrize("T,H", [(8, 256), (67, 1024), (512, 4096), (33, 8192)])
@pytest.mark.parametrize("with_res", [False, True])
def test_all_reduce_bias_residual_rmsnorm(emu_worlds, W, T, H, with_res):
    import tccl_b200 as tccl

    w = emu_worlds(W)
    x = w.from_parts([_rand((T, H), 4000 + r) for r in range(W)])
    bias, res, weight = _rand((H,), 1, 0.5), _rand((T, H), 2), _rand((H,), 3)
    rep = lambda t: [t for _ in range(W)]
    got = tccl.all_reduce_bias_residual_rmsnorm(x, rep(weight), rep(bias), rep(res), eps=1e-5,
                                                residual_out=True if with_res else None, world=w)
    torch.cuda.synchronize()
    w.check()
    y, h_out = got if with_res else (got, None)
    h = torch.stack([p.float() for p in x.parts]).sum(0) + bias.float() + res.float()
    if with_res:
        for r in range(W):
            assert bool(((h_out[r].float() - h).abs() <= h.abs() * 2 ** -8 + 1e-5).all())
        h = h.to(torch.bfloat16).float()  # the kernel normalises the rounded sum it stored
    ref = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + 1e-5) * weight.float()
    for r in range(W):
        err = (y[r].float() - ref).abs()
        assert bool((err <= ref.abs() * 2 ** -7 + 1e-3).all()), f"max err {err.max().item()}"
        assert torch.equal(y[r], y[0])


def test_fused_kernels_take_turns_on_the_staging_area(emu_worlds):
    """Pair and single-CTA GEMM -> reduce-scatter calls mixed with shape changes: the pair kernel runs
    without an entry barrier only after a call of its own kind; a change of user brings the barrier back."""
    import tccl_b200 as tccl

    W = 2
    w = emu_worlds(W)
    for M, N, K, variant in [(512, 256, 64, "pair"), (512, 256, 64, "pair"), (256, 256, 64, "single"),
                             (1024, 512, 128, "pair"), (512, 256, 64, "pair"), (512, 512, 64, "single"), (512, 256, 64, "pair")]:
        a = [_rand((M, K), 4000 + r + M) for r in range(W)]
        bt = [_rand((N, K), 5000 + r + N, 0.02) for r in range(W)]
        outs = tccl.gemm_reduce_scatter(a, bt, variant=variant, world=w)
        torch.cuda.synchronize()
        w.check()
        ref = sum(a[r].float() @ bt[r].float().t() for r in range(W))
        for r in range(W):
            exp = ref[r * (M // W):(r + 1) * (M // W)]
            assert bool(((outs[r].float() - exp).abs() <= exp.abs() * 2 ** -7 + 1e-2).all())


@pytest.mark.parametrize("variant", ["single", "pair"])
def test_all_gather_gemm_swiglu(emu_worlds, variant):
    import tccl_b200 as tccl
    from tccl_b200.ops.fused import pack_gate_up

    W, M, F, K = 2, 512, 256, 320
    w = emu_worlds(W)
    shards = [_rand((M // W, K), 10 + r) for r in range(W)]
    gate = [_rand((F, K), 20 + r, 0.05) for r in range(W)]
    up = [_rand((F, K), 30 + r, 0.05) for r in range(W)]
    packed = [pack_gate_up(gate[r], up[r]) for r in range(W)]
    outs, _ = tccl.all_gather_gemm(shards, packed, swiglu=True, variant=variant, world=w)
    torch.cuda.synchronize()
    w.check()
    a = torch.cat(shards).float()
    for r in range(W):
        ref = torch.nn.functional.silu(a @ gate[r].float().t()) * (a @ up[r].float().t())
        err = (outs[r].float() - ref).abs()
        assert outs[r].shape == (M, F)
        assert bool((err <= ref.abs() * 2 ** -7 + 2e-3).all()), err.max().item()


@pytest.mark.parametrize("W", [2, 4])
def test_tensor_parallel_mlp_matches_unsharded_fp32(emu_worlds, W):
    """Both forms of the TP MLP block against the unsharded fp32 block."""
    from tccl_b200.models import TensorParallelMLP

    w = emu_worlds(W)
    hidden, inter, T = 512, 1024, 128 * W
    fw = TensorParallelMLP.init_full_weights(hidden, inter, seed=4000)
    x = _rand((T, hidden), 77)
    ref = TensorParallelMLP.reference(x, fw)
    # emulated ranks: drive the fused ops with per-rank lists
    import tccl_b200 as tccl
    from tccl_b200.ops.fused import pack_gate_up

    blocks = [TensorParallelMLP(w, r, hidden, inter, full_weights=fw) for r in range(W)]
    shards = list(x.view(W, T // W, hidden).unbind(0))
    act, _ = tccl.all_gather_gemm(shards, [b.gate_up_packed for b in blocks], swiglu=True, world=w)
    outs = tccl.gemm_reduce_scatter(act, [b.down_w for b in blocks], world=w)
    torch.cuda.synchronize()
    w.check()
    got = torch.cat([o.float() for o in outs])
    err = (got - ref).abs()
    assert bool((err <= ref.abs() * 2 ** -6 + 3e-3).all()), err.max().item()
