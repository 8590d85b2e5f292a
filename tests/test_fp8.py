"""Block-scaled fp8 payloads: the CPU statement of the format everywhere, the CUDA kernels against
it on a GPU, and the exchange on the CPU/gloo backend with uneven shards."""

import pytest
import torch

from fast_ulysses_b200.ops import fp8


def test_cpu_round_trip_error_is_fp8_sized():
    torch.manual_seed(0)
    x = (torch.randn(2, 37, 5, 128) * torch.rand(2, 37, 5, 1) * 10).bfloat16()
    x[0, 0, 0] = 0  # an all-zero block keeps scale 1
    p = fp8.quantize(x)
    assert p.shape == (2, 37, 5, 144) and p.dtype == torch.uint8
    y = fp8.dequantize(p)
    amax = x.float().abs().amax(-1, keepdim=True).clamp_min(1e-30)
    assert ((y.float() - x.float()).abs() / amax).max() < 0.07  # e4m3: 3 mantissa bits
    assert torch.all(y[0, 0, 0] == 0)


@pytest.mark.gpu
def test_cuda_kernels_match_the_cpu_statement():
    torch.manual_seed(1)
    x = (torch.randn(3, 50, 4, 128, device="cuda") * 5).bfloat16()
    p_gpu = fp8.quantize(x)
    p_cpu = fp8.quantize(x.cpu())
    # scales are identical; payload bytes may differ by one rounding step where x/scale sits on a tie
    assert torch.equal(p_gpu[..., 128:132].cpu(), p_cpu[..., 128:132])
    diff = (fp8.dequantize(p_gpu).float().cpu() - fp8.dequantize(p_cpu).float()).abs()
    assert diff.max() <= 0.13 * x.float().abs().max().item()
    assert (diff > 0).float().mean() < 0.02
    y = fp8.dequantize(p_gpu)
    amax = x.float().abs().amax(-1, keepdim=True)
    assert ((y.float() - x.float()).abs() / amax).max() < 0.07
    assert torch.equal(fp8.dequantize(p_cpu.cuda()), fp8.dequantize(p_cpu).cuda())


def test_exchange_with_scales_over_gloo():
    from _dist import run_ranks

    run_ranks(3, "_gloo_workers", "fp8_exchange")
