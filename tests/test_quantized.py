"""All-reduce with the fp8 wire format, emulated ranks on one GPU, against an fp32 PyTorch sum and
against a plain PyTorch restatement of the same quantisation."""
import pytest
import torch

pytestmark = pytest.mark.gpu

CHUNK = 2048


def _q(x):
    """Per-chunk e4m3 quantisation as the kernel does it: value ~= fp8 * (absmax / 448)."""
    c = x.float().view(-1, CHUNK)
    scale = c.abs().amax(dim=1, keepdim=True).clamp_min(1e-30) * (1.0 / 448.0)
    q = (c * (1.0 / scale)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float()  # the kernel's conversion saturates
    return (q * scale).view(-1)


@pytest.mark.parametrize("W", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("n", [CHUNK, 5 * CHUNK, 64 * CHUNK, 1001 * CHUNK])
def test_quantized_all_reduce(emu_worlds, W, n):
    import tccl_b200 as tccl

    w = emu_worlds(W)
    parts = [(torch.randn(n, generator=torch.Generator().manual_seed(9000 + r)) * (1 + r)).to(torch.bfloat16)
             for r in range(W)]
    x = w.from_parts(parts)
    keep = [p.clone() for p in x.parts]
    for rep in range(2):
        out = tccl.quantized_all_reduce(x, world=w)
        torch.cuda.synchronize()
        w.check()
        ref = torch.stack([p.float() for p in x.parts]).sum(0)
        # the same arithmetic in PyTorch: quantise the partials, sum in fp32 in rank order, quantise the sum
        model = torch.zeros_like(ref)
        for r in range(W):
            model += _q(x[r])
        model = _q(model).to(torch.bfloat16)
        for r in range(W):
            assert torch.equal(out[r], out[0])          # every rank gets the same bits
            assert torch.equal(x[r], keep[r])           # the input is left alone
            # identical up to the rounding of 1/scale products (a different fp8 neighbour now and then)
            close = (out[r].float() - model.float()).abs() <= model.float().abs() * 2 ** -3 + 1e-6
            assert float(close.float().mean()) > 0.999 and bool(
                ((out[r].float() - model.float()).abs() <= ref.view(-1, CHUNK).abs().amax(1, keepdim=True).expand(-1, CHUNK).reshape(-1) * 2 ** -3 + 1e-6).all())
            # against the exact sum: two roundings to 3 mantissa bits, each within 2^-4 of a chunk maximum
            cmax = torch.stack([p.float().view(-1, CHUNK).abs().amax(1) for p in x.parts]).sum(0)
            bound = (cmax * 2 ** -4 + ref.view(-1, CHUNK).abs().amax(1) * 2 ** -4).unsqueeze(1).expand(-1, CHUNK).reshape(-1) * 1.05 + 1e-6
            assert bool(((out[r].float() - ref).abs() <= bound).all())


def test_quantized_all_reduce_rejects_bad_sizes(emu_worlds):
    import tccl_b200 as tccl

    w = emu_worlds(2)
    x = w.from_parts([torch.zeros(1000, dtype=torch.bfloat16) for _ in range(2)])
    with pytest.raises(ValueError):
        tccl.quantized_all_reduce(x, world=w)
    y = w.from_parts([torch.zeros(CHUNK, dtype=torch.float32) for _ in range(2)])
    with pytest.raises(TypeError):
        tccl.quantized_all_reduce(y, world=w)
