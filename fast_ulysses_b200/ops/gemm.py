"""bf16 GEMM on the tcgen05 tensor cores (csrc/kernels/gemm_sm100.cu).

``gemm_bf16(a, b)`` computes ``a @ b.T`` with fp32 accumulation in tensor memory; bias, GELU and a
residual add are fused into the epilogue. Both operands must have a contiguous last (K) axis.
``linear`` wraps it as a differentiable ``F.linear``: the backward runs two more of these GEMMs that
read dY, X and W as they lie in memory (``a_km`` / ``b_kn``), so every contraction of the block
stays on this kernel and nothing is transposed or copied.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _ckernels as ck

_err_words: dict[int, torch.Tensor] = {}


def error_word(device: torch.device) -> torch.Tensor:
    """One device word per GPU that kernels set when one of their bounded waits ran out."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _err_words:
        _err_words[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _err_words[idx]


def check_errors(device: torch.device | None = None) -> None:
    """Synchronising: raises if any tcgen05 kernel on this device gave up on a wait."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    code = int(error_word(device).item())
    if code:
        error_word(device).zero_()
        raise RuntimeError(f"fast_ulysses_b200: a tcgen05 kernel gave up on an internal wait (code {code})")


def _tma_ready(x: torch.Tensor) -> torch.Tensor:
    """A view of ``x`` whose rows are contiguous and start 16 bytes apart (copying if needed)."""
    if x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0:
        return x
    rows, cols = x.shape
    buf = torch.empty(rows, (cols + 7) // 8 * 8, dtype=x.dtype, device=x.device)
    out = buf[:, :cols]
    out.copy_(x)
    return out


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, *, bias: torch.Tensor | None = None,
              residual: torch.Tensor | None = None, act: int = 0, out: torch.Tensor | None = None,
              ctas: int = 0, a_km: bool = False, b_kn: bool = False, aux: torch.Tensor | None = None,
              store_pre: torch.Tensor | None = None, pair: bool | None = None) -> torch.Tensor:
    """``out[m, n] = act(a[m, :] . b[n, :] + bias[n]) + residual[m, n]`` (bf16 in, bf16 out).

    ``act``: 0 none, 1 GELU (tanh form), 2 GELU (erf form), 3 multiply by the derivative of the
    tanh-form GELU at ``aux[m, n]`` (the activation's backward, fused into the GEMM that produces
    its incoming gradient). ``store_pre`` (m, n) also receives the value before the activation.

    ``a_km`` / ``b_kn``: that operand is given with the contraction along its rows, ``a`` as
    ``(k, m)`` and ``b`` as ``(k, n)``; the kernel reads it as it lies in memory (no transposed
    copy), which is what the weight gradient ``dY^T X`` of a linear layer wants.

    ``pair``: run on pairs of CTAs (256 x 256 tiles, one tcgen05 MMA over two SMs) or on single
    CTAs (128 x 256); ``None`` leaves the choice to the library's default."""
    assert a.is_cuda and b.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.dim() == 2 and b.dim() == 2
    a, b = _tma_ready(a), _tma_ready(b)
    k, m = (a.shape[0], a.shape[1]) if a_km else (a.shape[1], a.shape[0])
    kb, n = (b.shape[0], b.shape[1]) if b_kn else (b.shape[1], b.shape[0])
    assert k == kb, (a.shape, b.shape, a_km, b_kn)
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    assert out.shape == (m, n) and out.stride(1) == 1 and out.dtype == torch.bfloat16
    g = ck.FuGemmArgs()
    g.a, g.b, g.c = a.data_ptr(), b.data_ptr(), out.data_ptr()
    g.m, g.n, g.k = m, n, k
    g.lda, g.ldb, g.ldc = a.stride(0), b.stride(0), out.stride(0)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == n and bias.is_contiguous()
        g.bias = bias.data_ptr()
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape == (m, n) and residual.stride(0) == out.stride(0)
        g.residual = residual.data_ptr()
    g.act = act
    for extra in (aux, store_pre):
        if extra is not None:
            assert extra.dtype == torch.bfloat16 and extra.shape == (m, n) and extra.stride() == out.stride()
    if aux is not None:
        g.aux = aux.data_ptr()
    if store_pre is not None:
        g.c_pre = store_pre.data_ptr()
    g.ctas = ctas
    g.flags = (1 if a_km else 0) | (2 if b_kn else 0) | (0 if pair is None else 4 if pair else 8)
    g.err = error_word(a.device).data_ptr()
    lib = ck.lib()
    ck.check(lib.fu_gemm_bf16(C.byref(g), ck.stream_ptr()))
    return out


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, residual):
        x2 = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.has_residual = residual is not None
        ctx.x_shape = x.shape
        r2 = residual.reshape(-1, weight.shape[0]) if residual is not None else None
        if r2 is not None and not r2.is_contiguous():
            r2 = r2.contiguous()
        y = gemm_bf16(x2, weight, bias=bias.float() if bias is not None else None, residual=r2)
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, weight = ctx.saved_tensors
        gy2 = gy.reshape(-1, gy.shape[-1]).contiguous()
        gx = gw = gb = None
        gr = gy if ctx.has_residual and ctx.needs_input_grad[3] else None
        if ctx.needs_input_grad[0]:
            # dX[m, k] = sum_n dY[m, n] W[n, k]: W as stored is the (contraction x output) operand
            gx = gemm_bf16(gy2, weight, b_kn=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            # dW[n, k] = sum_m dY[m, n] X[m, k]: both operands contract along their rows
            gw = gemm_bf16(gy2, x2, a_km=True, b_kn=True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = gy2.sum(0, dtype=torch.float32).to(gy.dtype)
        return gx, gw, gb, gr


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
           residual: torch.Tensor | None = None) -> torch.Tensor:
    """Differentiable ``x @ weight.T + bias (+ residual)`` on the tcgen05 GEMM (bf16); the residual is
    added in the GEMM's epilogue."""
    return _Linear.apply(x, weight, bias, residual)


class _LinearGelu(torch.autograd.Function):
    """``gelu_tanh(x @ w1.T + b1) @ w2.T + b2 (+ residual)``: the feed-forward of a transformer block as
    two GEMMs whose epilogues do everything else. Forward: GELU in the epilogue of the first GEMM,
    which also stores the pre-activation; residual in the epilogue of the second. Backward: the
    GELU's derivative is applied in the epilogue of the GEMM that produces its incoming gradient."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual):
        x2 = x.reshape(-1, x.shape[-1])
        pre = torch.empty(x2.shape[0], w1.shape[0], dtype=torch.bfloat16, device=x.device)
        h = gemm_bf16(x2, w1, bias=b1.float() if b1 is not None else None, act=1, store_pre=pre)
        r2 = residual.reshape(-1, w2.shape[0]) if residual is not None else None
        if r2 is not None and not r2.is_contiguous():
            r2 = r2.contiguous()
        y = gemm_bf16(h, w2, bias=b2.float() if b2 is not None else None, residual=r2)
        ctx.save_for_backward(x2, w1, w2, pre, h)
        ctx.flags = (b1 is not None, b2 is not None, residual is not None)
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, w1, w2, pre, h = ctx.saved_tensors
        has_b1, has_b2, has_res = ctx.flags
        gy2 = gy.reshape(-1, gy.shape[-1]).contiguous()
        gw2 = gemm_bf16(gy2, h, a_km=True, b_kn=True)
        gb2 = gy2.sum(0, dtype=torch.float32).to(gy.dtype) if has_b2 else None
        gpre = gemm_bf16(gy2, w2, b_kn=True, act=3, aux=pre)  # d(pre-activation) = (gy W2) * gelu'(pre)
        gw1 = gemm_bf16(gpre, x2, a_km=True, b_kn=True)
        gb1 = gpre.sum(0, dtype=torch.float32).to(gy.dtype) if has_b1 else None
        gx = gemm_bf16(gpre, w1, b_kn=True).view(ctx.x_shape)
        return gx, gw1, gb1, gw2, gb2, (gy if has_res else None)


def feed_forward(x, w1, b1, w2, b2, residual=None) -> torch.Tensor:
    """``gelu_tanh(x @ w1.T + b1) @ w2.T + b2 (+ residual)``, differentiable, four epilogue-fused GEMMs
    forward + backward-input and two weight-gradient GEMMs; no separate activation or add kernel."""
    return _LinearGelu.apply(x, w1, b1, w2, b2, residual)
