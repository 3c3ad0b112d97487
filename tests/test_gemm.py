"""tcgen05 GEMM against a PyTorch fp32 reference of the same bf16 operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (256, 512, 128), (384, 768, 1792),
                                   (200, 264, 72), (4096, 4096, 1792), (1000, 1792, 4096)])
def test_gemm_matches_fp32_reference(M, N, K):
    from tccl_b200.ops.gemm import gemm_bf16
    from tccl_b200.utils.lib import K as CONST

    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    a = torch.randn(M, K, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    bt = (torch.randn(N, K, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
    status = torch.zeros(CONST["TCCL_ST_WORDS"], dtype=torch.int32, device="cuda")
    out = gemm_bf16(a, bt, status=status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0, status.tolist()
    ref = a.float() @ bt.float().t()
    err = (out.float() - ref).abs()
    # fp32 accumulation, one rounding to bf16 (plus the order of the fp32 sums)
    bound = ref.abs() * 2 ** -8 + 1e-3 * (K ** 0.5) * 0.02
    assert bool((err <= bound).all()), f"max err {err.max().item()}, worst ratio {(err / bound).max().item()}"
