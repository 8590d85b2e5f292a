"""tcgen05 GEMM against a plain PyTorch fp32 statement of the same op."""

import pytest
import torch

from fast_ulysses_b200.ops import gemm

pytestmark = pytest.mark.gpu


def rel_err(got, want):
    return ((got.float() - want).norm() / want.norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 256), (300, 512, 256), (1000, 384, 320),
                                   (77, 40, 72), (2048, 1536, 1024), (256, 384, 213), (130, 72, 9)])
def test_gemm_matches_fp32(m, n, k):
    torch.manual_seed(m + n + k)
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = torch.randn(n, k, device="cuda").bfloat16()
    got = gemm.gemm_bf16(a, b)
    gemm.check_errors()
    want = a.float() @ b.float().t()
    assert got.shape == (m, n)
    assert rel_err(got, want) < 5e-3, rel_err(got, want)
    assert torch.allclose(got.float(), want, atol=0.5, rtol=2e-2)


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (128, 256, 256), (300, 520, 200), (1000, 384, 320), (77, 40, 72),
                                   (2048, 1536, 1024), (4096, 2048, 2048)])
def test_cta_pair_kernel_matches_fp32_and_the_single_cta_kernel_bit_for_bit(m, n, k):
    """256 x 256 tiles on pairs of CTAs (tcgen05 cta_group::2): the same products summed in the same
    order as the 128 x 256 single-CTA kernel, so not a bit may differ."""
    torch.manual_seed(m + n + k)
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = torch.randn(n, k, device="cuda").bfloat16()
    bias = torch.randn(n, device="cuda")
    got = gemm.gemm_bf16(a, b, bias=bias, act=1, pair=True)
    single = gemm.gemm_bf16(a, b, bias=bias, act=1, pair=False)
    gemm.check_errors()
    want = torch.nn.functional.gelu(a.float() @ b.float().t() + bias, approximate="tanh")
    assert rel_err(got, want) < 5e-3
    assert torch.equal(got, single)


@pytest.mark.parametrize("a_km,b_kn", [(True, True), (False, True), (True, False)])
def test_cta_pair_kernel_with_the_contraction_along_rows(a_km, b_kn):
    torch.manual_seed(11)
    m, n, k = 5120, 384, 9450
    a = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(n, k, device="cuda") * 0.5).bfloat16()
    got = gemm.gemm_bf16(a.t().contiguous() if a_km else a, b.t().contiguous() if b_kn else b, a_km=a_km, b_kn=b_kn,
                         pair=True)
    gemm.check_errors()
    assert rel_err(got, a.float() @ b.float().t()) < 5e-3


@pytest.mark.parametrize("act", [0, 1, 2])
def test_fused_epilogue(act):
    torch.manual_seed(act)
    m, n, k = 520, 776, 192
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = (torch.randn(n, k, device="cuda") * 0.1).bfloat16()
    bias = torch.randn(n, device="cuda")
    res = torch.randn(m, n, device="cuda").bfloat16()
    got = gemm.gemm_bf16(a, b, bias=bias, residual=res, act=act)
    gemm.check_errors()
    y = a.float() @ b.float().t() + bias
    if act == 1:
        y = torch.nn.functional.gelu(y, approximate="tanh")
    elif act == 2:
        y = torch.nn.functional.gelu(y)
    want = y + res.float()
    assert rel_err(got, want) < 6e-3, rel_err(got, want)


def test_strided_operands_and_many_tiles_per_cta():
    a_full = torch.randn(700, 1024, device="cuda").bfloat16()
    a = a_full[:, 128:640]  # leading dimension larger than k
    b = torch.randn(1024, 512, device="cuda").bfloat16()
    got = gemm.gemm_bf16(a, b, ctas=3)  # 6 x 4 tiles over 3 CTAs: accumulator buffers and ring wrap
    gemm.check_errors()
    assert rel_err(got, a.float() @ b.float().t()) < 5e-3


def test_linear_autograd():
    torch.manual_seed(0)
    x = torch.randn(3, 200, 256, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(384, 256, device="cuda") * 0.05).bfloat16().requires_grad_()
    bias = torch.randn(384, device="cuda").bfloat16().requires_grad_()
    y = gemm.linear(x, w, bias)
    gy = torch.randn_like(y)
    y.backward(gy)
    gemm.check_errors()
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, bias))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(gy.float())
    assert rel_err(y, yr.detach()) < 5e-3
    assert rel_err(x.grad, xr.grad) < 6e-3
    assert rel_err(w.grad, wr.grad) < 6e-3
    assert rel_err(bias.grad, br.grad) < 6e-3


@pytest.mark.parametrize("tokens", [9450, 75, 1001])
def test_linear_autograd_with_a_token_count_that_is_not_a_multiple_of_8(tokens):
    # the weight gradient contracts over the tokens: 75600 / 8 ranks = 9450 rows per rank
    torch.manual_seed(tokens)
    x = (torch.randn(tokens, 256, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(384, 256, device="cuda") * 0.1).bfloat16().requires_grad_()
    b = torch.randn(384, device="cuda").bfloat16().requires_grad_()
    y = gemm.linear(x, w, b)
    gy = torch.randn_like(y)
    y.backward(gy)
    gemm.check_errors()
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    torch.nn.functional.linear(xr, wr, br).backward(gy.float())
    assert rel_err(y, torch.nn.functional.linear(xr, wr, br)) < 1e-2
    assert rel_err(x.grad, xr.grad) < 1e-2 and rel_err(w.grad, wr.grad) < 1e-2 and rel_err(b.grad, br.grad) < 1e-2


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (300, 520, 200), (5120, 384, 9450), (72, 40, 1001)])
@pytest.mark.parametrize("a_km,b_kn", [(True, True), (False, True), (True, False)])
def test_operands_given_with_the_contraction_along_their_rows(m, n, k, a_km, b_kn):
    torch.manual_seed(m + n + k)
    a = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(n, k, device="cuda") * 0.5).bfloat16()
    want = a.float() @ b.float().t()
    if (a_km and m % 8) or (b_kn and n % 8):
        pytest.skip("a row pitch of the stored operand must be a multiple of 16 bytes")
    got = gemm.gemm_bf16(a.t().contiguous() if a_km else a, b.t().contiguous() if b_kn else b, a_km=a_km, b_kn=b_kn)
    gemm.check_errors()
    assert rel_err(got, want) < 5e-3


def test_feed_forward_epilogues_match_pytorch():
    """GELU forward in the first GEMM's epilogue (which also stores the pre-activation), its
    derivative in the epilogue of the GEMM that produces its incoming gradient, bias and residual in
    epilogues: against the same feed-forward in fp32 PyTorch, values and all five gradients."""
    torch.manual_seed(3)
    m, hidden, ffn = 300, 256, 520
    x = torch.randn(2, m // 2, hidden, device="cuda").bfloat16().requires_grad_()
    res = torch.randn(2, m // 2, hidden, device="cuda").bfloat16().requires_grad_()
    w1 = (torch.randn(ffn, hidden, device="cuda") * 0.06).bfloat16().requires_grad_()
    b1 = (torch.randn(ffn, device="cuda") * 0.1).bfloat16().requires_grad_()
    w2 = (torch.randn(hidden, ffn, device="cuda") * 0.06).bfloat16().requires_grad_()
    b2 = (torch.randn(hidden, device="cuda") * 0.1).bfloat16().requires_grad_()
    y = gemm.feed_forward(x, w1, b1, w2, b2, residual=res)
    dy = torch.randn_like(y)
    y.backward(dy)
    gemm.check_errors()
    ref = [t.detach().float().requires_grad_() for t in (x, w1, b1, w2, b2, res)]
    h = torch.nn.functional.gelu(torch.nn.functional.linear(ref[0], ref[1], ref[2]), approximate="tanh")
    yr = torch.nn.functional.linear(h, ref[3], ref[4]) + ref[5]
    yr.backward(dy.float())
    assert rel_err(y, yr) < 1e-2, rel_err(y, yr)
    for name, got, want in zip(("x", "w1", "b1", "w2", "b2", "residual"), (x, w1, b1, w2, b2, res), ref):
        assert rel_err(got.grad, want.grad) < 2.5e-2, (name, rel_err(got.grad, want.grad))


def test_linear_with_residual_in_the_epilogue():
    torch.manual_seed(4)
    x = torch.randn(130, 192, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(264, 192, device="cuda") * 0.07).bfloat16().requires_grad_()
    r = torch.randn(130, 264, device="cuda").bfloat16().requires_grad_()
    y = gemm.linear(x, w, None, residual=r)
    y.backward(torch.ones_like(y))
    gemm.check_errors()
    want = x.detach().float() @ w.detach().float().t() + r.detach().float()
    assert rel_err(y, want) < 1e-2
    assert torch.equal(r.grad, torch.ones_like(r))
