"""The fused mode-1 path: the output projection whose A operand is pulled from the peers'
attention outputs inside the same kernel (csrc/kernels/gemm_sm100.cu:fu_pull_outproj)."""

from __future__ import annotations

import ctypes as C

import torch

from . import _ckernels as ck
from .gemm import error_word


def pull_outproj_raw(w: torch.Tensor, out: torch.Tensor, gather: torch.Tensor, ready: torch.Tensor, *, s_local: int,
                     seq_off: int, s_total: int, head_splits: list[int], rank: int, peer_o: list[int],
                     ctrl: list[int], o_bytes: int, bias: torch.Tensor | None = None,
                     residual: torch.Tensor | None = None, flags: int = 0, timeout_ms: int = 10000,
                     ctas: int = 0) -> torch.Tensor:
    """out[m, n] = A[m, :] . w[n, :] (+ bias + residual) with A gathered from ``peer_o`` (each a
    (b, s_total, head_splits[p], 128) bf16 buffer address with ``o_bytes`` bytes behind it: the
    launcher refuses a shape whose loads would leave a peer's buffer). ``gather`` is (m, heads*128)
    bf16 scratch; afterwards it holds the gathered A (the backward reuses it)."""
    m, n = out.shape
    heads = sum(head_splits)
    assert w.shape == (n, heads * 128) and w.dtype == torch.bfloat16 and w.stride(1) == 1
    assert gather.shape == (m, heads * 128) and gather.is_contiguous() and gather.dtype == torch.bfloat16
    assert ready.dtype == torch.int32 and ready.numel() >= ((m + 127) // 128) * len(head_splits)
    a = ck.FuPullArgs()
    a.w, a.c, a.m, a.n, a.ldw, a.ldc = w.data_ptr(), out.data_ptr(), m, n, w.stride(0), out.stride(0)
    if bias is not None:
        assert bias.dtype == torch.float32
        a.bias = bias.data_ptr()
    if residual is not None:
        assert residual.shape == out.shape and residual.stride(0) == out.stride(0)
        a.residual = residual.data_ptr()
    a.s_local, a.seq_off, a.s_total = s_local, seq_off, s_total
    a.rank, a.world = rank, len(head_splits)
    for p, h in enumerate(head_splits):
        a.head_splits[p] = h
        a.peer_o[p] = peer_o[p]
        a.peer_ctrl[p] = ctrl[p]
    a.gather, a.ready = gather.data_ptr(), ready.data_ptr()
    a.o_bytes, a.gather_bytes, a.ready_words = o_bytes, gather.numel() * 2, ready.numel()
    a.flags, a.timeout_ms, a.ctas = flags, timeout_ms, ctas
    a.err = error_word(out.device).data_ptr()
    ck.check(ck.lib().fu_pull_outproj(C.byref(a), ck.stream_ptr()))
    return out
