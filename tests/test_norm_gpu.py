"""The one-kernel LayerNorm (forward and backward) against PyTorch in fp32."""

import pytest
import torch

from fast_ulysses_b200.ops.norm import layer_norm

pytestmark = pytest.mark.gpu


def rel_err(got, want):
    return ((got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("shape", [(1, 37, 256), (2, 130, 5120), (3, 8)])
def test_layer_norm_forward_and_backward(shape):
    torch.manual_seed(sum(shape))
    x = (torch.randn(*shape, device="cuda") * 3 + 1.5).bfloat16().requires_grad_()
    y = layer_norm(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = torch.nn.functional.layer_norm(xr, (shape[-1],), eps=1e-6)
    yr.backward(dy.float())
    assert rel_err(y, yr) < 1e-2, rel_err(y, yr)
    assert rel_err(x.grad, xr.grad) < 1.5e-2, rel_err(x.grad, xr.grad)


def test_layer_norm_reads_a_row_strided_view_in_place():
    torch.manual_seed(1)
    big = torch.randn(64, 512, device="cuda").bfloat16()
    x = big[:, :256]  # rows 1024 bytes apart, 512 bytes used
    y = layer_norm(x)
    want = torch.nn.functional.layer_norm(x.float(), (256,), eps=1e-6)
    assert rel_err(y, want) < 1e-2
