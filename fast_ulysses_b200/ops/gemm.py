"""bf16 GEMM on the tcgen05 tensor cores (csrc/kernels/gemm_sm100.cu).

``gemm_bf16(a, b)`` computes ``a @ b.T`` with fp32 accumulation in tensor memory; bias, GELU and a
residual add are fused into the epilogue. Both operands must have a contiguous last (K) axis.
``linear`` wraps it as a differentiable ``F.linear``: the backward runs two more of these GEMMs on
transposed copies, so every contraction of the block stays on this kernel.
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


def transpose_for_gemm(x: torch.Tensor) -> torch.Tensor:
    """``x.t()`` materialised with a 16-byte row pitch, ready to be a K-major GEMM operand."""
    return _tma_ready(x.t())


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, *, bias: torch.Tensor | None = None,
              residual: torch.Tensor | None = None, act: int = 0, out: torch.Tensor | None = None,
              ctas: int = 0, a_km: bool = False, b_kn: bool = False) -> torch.Tensor:
    """``out[m, n] = act(a[m, :] . b[n, :] + bias[n]) + residual[m, n]`` (bf16 in, bf16 out).

    ``a_km`` / ``b_kn``: that operand is given with the contraction along its rows, ``a`` as
    ``(k, m)`` and ``b`` as ``(k, n)``; the kernel reads it as it lies in memory (no transposed
    copy), which is what the weight gradient ``dY^T X`` of a linear layer wants."""
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
    g.ctas = ctas
    g.flags = (1 if a_km else 0) | (2 if b_kn else 0)
    g.err = error_word(a.device).data_ptr()
    lib = ck.lib()
    ck.check(lib.fu_gemm_bf16(C.byref(g), ck.stream_ptr()))
    return out


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        y = gemm_bf16(x2, weight, bias=bias.float() if bias is not None else None)
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, weight = ctx.saved_tensors
        gy2 = gy.reshape(-1, gy.shape[-1]).contiguous()
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            # dX[m, k] = sum_n dY[m, n] W[n, k]: W as stored is the (contraction x output) operand
            gx = gemm_bf16(gy2, weight, b_kn=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            # dW[n, k] = sum_m dY[m, n] X[m, k]: both operands contract along their rows
            gw = gemm_bf16(gy2, x2, a_km=True, b_kn=True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = gy2.sum(0, dtype=torch.float32).to(gy.dtype)
        return gx, gw, gb


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """Differentiable ``x @ weight.T + bias`` on the tcgen05 GEMM (bf16)."""
    return _Linear.apply(x, weight, bias)
