"""The shared error bounds accept what the arithmetic can produce and reject a dropped partial."""
import torch

from tccl_b200.utils.numerics import allreduce_rmsnorm_check


def _case(W=4, T=16, H=256, seed=0):
    g = torch.Generator().manual_seed(seed)
    parts = [torch.randn(T, H, generator=g).to(torch.bfloat16) for _ in range(W)]
    bias, resid, wn = (torch.randn(H, generator=g) * 0.5).bfloat16(), torch.randn(T, H, generator=g).bfloat16(), torch.randn(H, generator=g).bfloat16()
    s = sum(p.float() for p in parts)
    return parts, bias, resid, wn, s


def _norm(h_out, wn, eps=1e-5):
    hb = h_out.float()
    return (hb * torch.rsqrt((hb * hb).mean(-1, keepdim=True) + eps) * wn.float()).to(torch.bfloat16)


def test_round_to_nearest_sum_passes_both_bounds():
    parts, bias, resid, wn, s = _case()
    h_out = (s + bias.float() + resid.float()).to(torch.bfloat16)
    for nvls in (False, True):
        ok, worst = allreduce_rmsnorm_check(_norm(h_out, wn), h_out, s, bias, resid, wn, 1e-5, 4, nvls)
        assert ok and worst <= 1.0


def test_switch_style_rounding_of_the_partial_sum_needs_the_nvls_bound():
    parts, bias, resid, wn, s = _case(seed=1)
    s_trunc = (s.view(torch.int32) & ~0xFFFF).view(torch.float32)  # bf16 by truncation: up to one ulp off
    h_out = (s_trunc + bias.float() + resid.float()).to(torch.bfloat16)
    ok, _ = allreduce_rmsnorm_check(_norm(h_out, wn), h_out, s, bias, resid, wn, 1e-5, 4, True)
    assert ok
    ok_p2p, worst = allreduce_rmsnorm_check(_norm(h_out, wn), h_out, s, bias, resid, wn, 1e-5, 4, False)
    assert not ok_p2p and worst > 1.0


def test_a_dropped_partial_fails():
    parts, bias, resid, wn, s = _case(seed=2)
    h_bad = (s - parts[3].float() + bias.float() + resid.float()).to(torch.bfloat16)
    ok, worst = allreduce_rmsnorm_check(_norm(h_bad, wn), h_bad, s, bias, resid, wn, 1e-5, 4, True)
    assert not ok and worst > 10
