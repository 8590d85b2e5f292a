"""Flash attention on the tcgen05 tensor cores (csrc/kernels/fmha_fwd_sm100.cu, fmha_bwd_sm100.cu).

Tensors use the ``(batch, seq, heads, 128)`` layout of the all-to-all windows; any view whose last
axis is contiguous and whose other strides are multiples of 8 elements is read in place.
"""

from __future__ import annotations

import ctypes as C
import math

import torch

from . import _ckernels as ck
from .gemm import error_word


def _strides(t: torch.Tensor):
    assert t.dim() == 4 and t.shape[-1] == 128 and t.stride(3) == 1 and t.dtype == torch.bfloat16, (t.shape, t.stride())
    return t.stride(1), t.stride(2), t.stride(0)


def _fill(a, q, k, v, o):
    b, sq, h, _ = q.shape
    a.q, a.k, a.v, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    a.batch, a.heads, a.seq_q, a.seq_kv, a.head_dim = b, h, sq, k.shape[1], 128
    a.q_row, a.q_head, a.q_batch = _strides(q)
    a.k_row, a.k_head, a.k_batch = _strides(k)
    a.v_row, a.v_head, a.v_batch = _strides(v)
    a.o_row, a.o_head, a.o_batch = _strides(o)
    a.err = error_word(q.device).data_ptr()


def fmha_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float | None = None,
             out: torch.Tensor | None = None, ctas: int = 0, poly: int | None = None,
             trace: torch.Tensor | None = None):
    """``softmax(q k^T * scale) v`` for (b, s, h, 128) bf16 tensors. Returns ``(o, lse)`` with
    ``lse`` of shape (b, h, s_q), fp32, natural log. ``poly`` (0, 2, 4 or 6) overrides how many of
    every 16 exponential pairs are computed on the FMA pipe instead of the special-function unit.
    ``trace`` (int64[256] on the device) selects the instrumented build of the kernel: CTA 0 stores the
    SM clock of 32 pipeline events for kv steps 64..71 of its first item."""
    b, sq, h, d = q.shape
    assert k.shape == v.shape and k.shape[0] == b and k.shape[2] == h and d == 128
    o = out if out is not None else torch.empty(b, sq, h, d, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(b, h, sq, dtype=torch.float32, device=q.device)
    a = ck.FuFmhaArgs()
    _fill(a, q, k, v, o)
    a.lse = lse.data_ptr()
    a.scale = scale if scale is not None else 1.0 / math.sqrt(d)
    a.ctas = ctas
    if poly is not None:
        a.flags = 0x1000 | ((poly & 15) << 8)  # FU_FMHA_POLY(poly)
    if trace is not None:
        assert trace.dtype == torch.int64 and trace.numel() >= 256 and trace.is_cuda
        a.trace = trace.data_ptr()
    ck.check(ck.lib().fu_fmha_fwd(C.byref(a), ck.stream_ptr()))
    return o, lse


def attention_reference(q, k, v, scale=None):
    """fp32 PyTorch statement on (b, s, h, d) tensors; returns (o, lse)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    lse = torch.logsumexp(s, dim=-1)
    o = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, dim=-1), v.float())
    return o, lse


def fmha_bwd(q, k, v, o, lse, d_o, *, scale: float | None = None, ctas: int = 0, out=None,
             deterministic: bool = False, trace: torch.Tensor | None = None):
    """Gradients of ``fmha_fwd``. All tensors (b, s, h, 128) bf16; ``d_o`` must share ``o``'s
    strides. Returns ``(dq, dk, dv)`` shaped and strided like q, k, v (dense). The default is one
    software-pipelined pass that sums dQ over the K/V blocks with fp32 reductions (dK and dV are
    bit-reproducible, dQ to rounding); ``deterministic=True`` runs two passes without atomics
    (dK/dV with the K/V block stationary, then dQ with the query rows stationary) at about 1.5x
    the time."""
    b, sq, h, d = q.shape
    if d_o.stride() != o.stride():
        d_o = d_o.contiguous()
        o = o.contiguous()
    if out is not None:
        dq, dk, dv = out  # dense (b, s, h, 128) tensors provided by the caller
        assert dq.is_contiguous() and dk.is_contiguous() and dv.is_contiguous()
    else:
        dq = torch.empty(b, sq, h, d, dtype=torch.bfloat16, device=q.device)
        dk = torch.empty(b, k.shape[1], h, d, dtype=torch.bfloat16, device=q.device)
        dv = torch.empty_like(dk)
    # the launcher addresses dq/dk/dv with the strides of q/k/v: hand it dense q/k/v views
    qc, kc, vc = (t if t.is_contiguous() else t.contiguous() for t in (q, k, v))
    sq_pad = (sq + 127) // 128 * 128
    stats = torch.empty(2 * b * h * sq_pad, dtype=torch.float32, device=q.device)
    dq_acc = None if deterministic else torch.empty(b, sq, h, d, dtype=torch.float32, device=q.device)
    a = ck.FuFmhaArgs()
    _fill(a, qc, kc, vc, o)
    a.lse = lse.data_ptr()
    a.scale = scale if scale is not None else 1.0 / math.sqrt(d)
    a.ctas = ctas
    a.d_o, a.dq, a.dk, a.dv = d_o.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.delta = stats.data_ptr()
    if dq_acc is not None:
        a.dq_acc = dq_acc.data_ptr()
    a.flags = 1 if deterministic else 0
    if trace is not None:  # int64[128] on the device: SM clock of 16 pipeline events for 8 blocks of CTA 0
        a.trace = trace.data_ptr()
    ck.check(ck.lib().fu_fmha_bwd(C.byref(a), ck.stream_ptr()))
    return dq, dk, dv


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale):
        o, lse = fmha_fwd(q, k, v, scale=scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = fmha_bwd(q, k, v, o, lse, d_o.contiguous() if not d_o.is_contiguous() else d_o, scale=ctx.scale)
        return dq, dk, dv, None


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None) -> torch.Tensor:
    """Differentiable non-causal attention on (b, s, h, 128) bf16 tensors (tcgen05 fwd and bwd)."""
    return _Attention.apply(q, k, v, scale)
