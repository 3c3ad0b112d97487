"""tcgen05 GEMM against a PyTorch fp32 reference of the same bf16 operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("variant", ["single", "pair"])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (256, 512, 128), (384, 768, 1792),
                                   (200, 264, 72), (4096, 4096, 1792), (1000, 1792, 4096), (4096, 1792, 4096),
                                   (2304, 1280, 512), (8, 8, 8)])
def test_gemm_matches_fp32_reference(M, N, K, variant):
    from tccl_b200.ops.gemm import gemm_bf16
    from tccl_b200.utils.lib import K as CONST

    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    a = torch.randn(M, K, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    bt = (torch.randn(N, K, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
    status = torch.zeros(CONST["TCCL_ST_WORDS"], dtype=torch.int32, device="cuda")
    out = gemm_bf16(a, bt, status=status, variant=variant)
    torch.cuda.synchronize()
    assert int(status[0]) == 0, status.tolist()
    ref = a.float() @ bt.float().t()
    err = (out.float() - ref).abs()
    # fp32 accumulation, one rounding to bf16 (plus the order of the fp32 sums)
    bound = ref.abs() * 2 ** -8 + 1e-3 * (K ** 0.5) * 0.02
    assert bool((err <= bound).all()), f"max err {err.max().item()}, worst ratio {(err / bound).max().item()}"


@pytest.mark.parametrize("ctas", [2, 6, 20, 148])
def test_pair_gemm_tail_wave_split_for_any_grid(ctas):
    """The last partial wave is cut into half tiles: every number of pairs must still cover every
    output element exactly once."""
    from tccl_b200.ops.gemm import gemm_bf16

    M, N, K = 1280, 1536, 256   # 5 x 6 = 30 tiles of 256 x 256
    g = torch.Generator(device="cuda").manual_seed(ctas)
    a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    bt = (torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    gemm_bf16(a, bt, out=out, ctas=ctas, variant="pair")
    torch.cuda.synchronize()
    ref = a.float() @ bt.float().t()
    assert bool(((out.float() - ref).abs() <= ref.abs() * 2 ** -8 + 2e-3).all())
