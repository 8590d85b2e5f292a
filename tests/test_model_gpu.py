"""The fused sequence-parallel attention block and the DiT stack on ONE GPU (a single-rank group
runs every fused kernel: scatter epilogue, attention, pull prologue) against plain PyTorch."""

import pytest
import torch

import fast_ulysses_b200 as fu
from fast_ulysses_b200.models.attention import UlyssesSelfAttention, reference_attention
from fast_ulysses_b200.models.dit import DiTStack, reference_forward
from fast_ulysses_b200.ops import gemm

pytestmark = pytest.mark.gpu


def rel_err(got, want):
    return ((got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-12)).item()


def test_attention_block_forward_backward_single_rank():
    torch.manual_seed(0)
    g = fu.UlyssesGroup(device="cuda")
    grid, hidden, heads = (3, 10, 16), 512, 4  # 480 tokens
    attn = UlyssesSelfAttention(g, hidden, heads, grid=grid)
    with torch.no_grad():
        attn.gamma_q.add_(0.1 * torch.randn_like(attn.gamma_q))
        attn.gamma_k.add_(0.1 * torch.randn_like(attn.gamma_k))
        attn.b_o.add_(0.1 * torch.randn_like(attn.b_o.float()).bfloat16())
    x = torch.randn(1, 480, hidden, device="cuda").bfloat16().requires_grad_()
    y = attn(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    gemm.check_errors()
    g.check()

    params = [attn.w_qkv, attn.gamma_q, attn.gamma_k, attn.w_o, attn.b_o]
    xr = x.detach().float().requires_grad_()
    pr = [p.detach().float().requires_grad_() for p in params]
    yr = reference_attention(xr, pr[0], pr[1], pr[2], pr[3], pr[4], heads, grid)
    yr.backward(dy.float())
    assert rel_err(y, yr) < 2e-2, rel_err(y, yr)
    assert rel_err(x.grad, xr.grad) < 3e-2, ("dx", rel_err(x.grad, xr.grad))
    for name, p, r in zip(("w_qkv", "gamma_q", "gamma_k", "w_o", "b_o"), params, pr):
        assert rel_err(p.grad, r.grad) < 4e-2, (name, rel_err(p.grad, r.grad))
    g.destroy()


def test_dit_stack_single_rank():
    torch.manual_seed(1)
    g = fu.UlyssesGroup(device="cuda")
    grid = (2, 8, 16)  # 256 tokens
    stack = DiTStack(g, depth=2, hidden=256, heads=2, ffn=512, grid=grid)
    x = torch.randn(1, 256, 256, device="cuda").bfloat16().requires_grad_()
    y = stack(x)
    y.float().pow(2).mean().backward()
    gemm.check_errors()
    xr = x.detach().float().requires_grad_()
    yr = reference_forward(stack, xr)
    yr.pow(2).mean().backward()
    assert rel_err(y, yr) < 3e-2, rel_err(y, yr)
    assert rel_err(x.grad, xr.grad) < 6e-2, rel_err(x.grad, xr.grad)
    g.destroy()


def test_backward_after_a_later_forward_is_refused():
    """The block keeps q, k, v and the attention output in its symmetric buffers: a backward for a
    forward that a later forward has overwritten must raise, not return another call's gradients."""
    torch.manual_seed(2)
    g = fu.UlyssesGroup(device="cuda")
    grid, hidden, heads = (2, 8, 16), 256, 2
    attn = UlyssesSelfAttention(g, hidden, heads, grid=grid)
    x1 = torch.randn(1, 256, hidden, device="cuda").bfloat16().requires_grad_()
    x2 = torch.randn(1, 256, hidden, device="cuda").bfloat16().requires_grad_()
    y1 = attn(x1)
    y2 = attn(x2)
    with pytest.raises(RuntimeError, match="forward ran again"):
        y1.sum().backward()
    y2.sum().backward()  # the latest forward still owns the buffers
    # forward, backward, forward, backward (gradient accumulation) is the supported order
    attn.zero_grad()
    attn(x1).sum().backward()
    first = attn.w_o.grad.clone()
    attn(x1).sum().backward()
    assert torch.allclose(attn.w_o.grad.float(), 2 * first.float(), rtol=2e-2, atol=1e-3)
    gemm.check_errors()
    g.destroy()
