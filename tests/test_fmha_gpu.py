"""tcgen05 flash attention against an fp32 PyTorch statement (small S) and torch SDPA (larger S)."""

import pytest
import torch

from fast_ulysses_b200.ops import attention, gemm

pytestmark = pytest.mark.gpu


def rel_err(got, want):
    return ((got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("b,h,sq,skv", [(1, 1, 128, 128), (1, 1, 256, 256), (1, 2, 256, 384), (2, 3, 300, 500),
                                        (1, 2, 1000, 1111), (1, 1, 77, 1)])
def test_forward_matches_fp32(b, h, sq, skv):
    torch.manual_seed(sq + skv)
    q = torch.randn(b, sq, h, 128, device="cuda").bfloat16()
    k = torch.randn(b, skv, h, 128, device="cuda").bfloat16()
    v = torch.randn(b, skv, h, 128, device="cuda").bfloat16()
    o, lse = attention.fmha_fwd(q, k, v)
    gemm.check_errors()
    o_ref, lse_ref = attention.attention_reference(q, k, v)
    assert rel_err(o, o_ref) < 1.5e-2, rel_err(o, o_ref)
    assert torch.allclose(lse, lse_ref, atol=2e-2, rtol=1e-3), (lse - lse_ref).abs().max().item()


@pytest.mark.parametrize("poly", [0, 2, 4, 6])
def test_forward_exponentials_split_between_the_pipes(poly):
    """Part of the exponentials as a cubic on the FMA pipe: same result within bf16 rounding,
    for scores whose spread reaches the clamp of the cubic's argument."""
    torch.manual_seed(11)
    q = (torch.randn(1, 300, 2, 128, device="cuda") * 3).bfloat16()
    k = (torch.randn(1, 700, 2, 128, device="cuda") * 3).bfloat16()
    v = torch.randn(1, 700, 2, 128, device="cuda").bfloat16()
    o, lse = attention.fmha_fwd(q, k, v, poly=poly)
    gemm.check_errors()
    o_ref, lse_ref = attention.attention_reference(q, k, v)
    assert rel_err(o, o_ref) < 1.5e-2, rel_err(o, o_ref)
    assert torch.allclose(lse, lse_ref, atol=2e-2, rtol=1e-3), (lse - lse_ref).abs().max().item()


def test_large_scores_exercise_the_lazy_rescale():
    torch.manual_seed(3)
    q = (torch.randn(1, 256, 1, 128, device="cuda") * 4).bfloat16()
    k = (torch.randn(1, 2048, 1, 128, device="cuda") * 4).bfloat16()
    k[:, 1500:] *= 3  # the maximum keeps growing late in the kv loop
    v = torch.randn(1, 2048, 1, 128, device="cuda").bfloat16()
    o, lse = attention.fmha_fwd(q, k, v)
    gemm.check_errors()
    o_ref, lse_ref = attention.attention_reference(q, k, v)
    assert rel_err(o, o_ref) < 2e-2, rel_err(o, o_ref)
    assert torch.allclose(lse, lse_ref, atol=5e-2, rtol=1e-3)


def test_window_layout_views_and_many_items_per_cta():
    """q, k, v as slices of one packed (b, s, 3, h, d) buffer; few CTAs so that each loops over items."""
    torch.manual_seed(5)
    packed = torch.randn(1, 640, 3, 5, 128, device="cuda").bfloat16()
    q, k, v = packed[:, :, 0], packed[:, :, 1], packed[:, :, 2]
    o, lse = attention.fmha_fwd(q, k, v, ctas=2)
    gemm.check_errors()
    o_ref, lse_ref = attention.attention_reference(q, k, v)
    assert rel_err(o, o_ref) < 1.5e-2
    assert torch.allclose(lse, lse_ref, atol=2e-2, rtol=1e-3)


def test_against_sdpa_longer_sequence():
    torch.manual_seed(9)
    q = torch.randn(1, 4096, 4, 128, device="cuda").bfloat16()
    k = torch.randn(1, 4096, 4, 128, device="cuda").bfloat16()
    v = torch.randn(1, 4096, 4, 128, device="cuda").bfloat16()
    o, _ = attention.fmha_fwd(q, k, v)
    gemm.check_errors()
    ref = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    assert rel_err(o, ref.transpose(1, 2)) < 1.5e-2


@pytest.mark.parametrize("b,h,sq,skv", [(1, 1, 128, 128), (1, 2, 256, 384), (2, 2, 300, 500), (1, 1, 1000, 777)])
def test_backward_matches_fp32_autograd(b, h, sq, skv):
    torch.manual_seed(sq * 3 + skv)
    q = torch.randn(b, sq, h, 128, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(b, skv, h, 128, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(b, skv, h, 128, device="cuda").bfloat16().requires_grad_()
    o = attention.attention(q, k, v)
    d_o = torch.randn_like(o)
    o.backward(d_o)
    gemm.check_errors()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    o_ref, _ = attention.attention_reference(qr, kr, vr)
    o_ref.backward(d_o.float())
    assert rel_err(q.grad, qr.grad) < 2e-2, ("dq", rel_err(q.grad, qr.grad))
    assert rel_err(k.grad, kr.grad) < 2e-2, ("dk", rel_err(k.grad, kr.grad))
    assert rel_err(v.grad, vr.grad) < 2e-2, ("dv", rel_err(v.grad, vr.grad))


@pytest.mark.parametrize("b,h,sq,skv", [(1, 1, 128, 128), (1, 2, 256, 384), (2, 2, 300, 500), (1, 1, 1000, 777)])
def test_backward_deterministic_two_pass(b, h, sq, skv):
    torch.manual_seed(sq + skv)
    q = torch.randn(b, sq, h, 128, device="cuda").bfloat16()
    k = torch.randn(b, skv, h, 128, device="cuda").bfloat16()
    v = torch.randn(b, skv, h, 128, device="cuda").bfloat16()
    o, lse = attention.fmha_fwd(q, k, v)
    d_o = torch.randn_like(o)
    dq, dk, dv = attention.fmha_bwd(q, k, v, o, lse, d_o, deterministic=True)
    again = attention.fmha_bwd(q, k, v, o, lse, d_o, deterministic=True)
    gemm.check_errors()
    assert all(torch.equal(x, y) for x, y in zip((dq, dk, dv), again))
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    o_ref, _ = attention.attention_reference(qr, kr, vr)
    o_ref.backward(d_o.float())
    assert rel_err(dq, qr.grad) < 2e-2, ("dq", rel_err(dq, qr.grad))
    assert rel_err(dk, kr.grad) < 2e-2, ("dk", rel_err(dk, kr.grad))
    assert rel_err(dv, vr.grad) < 2e-2, ("dv", rel_err(dv, vr.grad))


@pytest.mark.parametrize("deterministic", [False, True], ids=["single-pass", "two-pass"])
def test_backward_many_blocks_per_cta(deterministic):
    torch.manual_seed(1)
    q = torch.randn(1, 640, 3, 128, device="cuda").bfloat16()
    k = torch.randn(1, 900, 3, 128, device="cuda").bfloat16()
    v = torch.randn(1, 900, 3, 128, device="cuda").bfloat16()
    o, lse = attention.fmha_fwd(q, k, v)
    d_o = torch.randn_like(o)
    dq, dk, dv = attention.fmha_bwd(q, k, v, o, lse, d_o, ctas=2, deterministic=deterministic)
    gemm.check_errors()
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    o_ref, _ = attention.attention_reference(qr, kr, vr)
    o_ref.backward(d_o.float())
    assert rel_err(dq, qr.grad) < 2e-2 and rel_err(dk, kr.grad) < 2e-2 and rel_err(dv, vr.grad) < 2e-2
