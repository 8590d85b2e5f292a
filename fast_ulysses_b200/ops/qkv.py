"""The fused mode-0 path: QKV projection + per-head RMSNorm + 3D RoPE + head scatter in one kernel.

``qkv_rope_scatter_raw`` launches csrc/kernels/gemm_sm100.cu:fu_qkv_rope_scatter on raw window
pointers (this is what single-GPU tests use, with fake peers on one device). The differentiable,
group-aware wrapper lives in :mod:`fast_ulysses_b200.models.attention`.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _ckernels as ck
from .gemm import error_word

HEAD_DIM = 128


def qkv_rope_scatter_raw(x: torch.Tensor, w: torch.Tensor, rope: torch.Tensor, gamma_q: torch.Tensor,
                         gamma_k: torch.Tensor, *, heads: int, s_local: int, seq_off: int, s_total: int,
                         head_splits: list[int], rank: int, win_q: list[int], win_k: list[int], win_v: list[int],
                         ctrl: list[int], win_bytes: int, eps: float = 1e-6, flags: int = 0,
                         timeout_ms: int = 10000, ctas: int = 0) -> None:
    """x: (b * s_local, hidden) bf16, w: (3 * heads * 128, hidden) bf16 (rows: q heads, k heads,
    v heads). Each rank's q/k/v window has layout (b, s_total, head_splits[p], 128) bf16 and
    ``win_bytes`` bytes behind its base; the launcher refuses a shape whose stores would leave it."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
    assert w.shape[0] == 3 * heads * HEAD_DIM and w.shape[1] == x.shape[1]
    assert rope.dtype == torch.float32 and rope.shape == (s_local, HEAD_DIM // 2, 2) and rope.is_contiguous()
    world = len(head_splits)
    a = ck.FuQkvArgs()
    a.x, a.w = x.data_ptr(), w.data_ptr()
    a.m, a.k, a.ldx, a.ldw = x.shape[0], x.shape[1], x.stride(0), w.stride(0)
    a.heads = heads
    a.s_local, a.seq_off, a.s_total = s_local, seq_off, s_total
    a.rope, a.gamma_q, a.gamma_k = rope.data_ptr(), gamma_q.data_ptr(), gamma_k.data_ptr()
    assert gamma_q.dtype == torch.float32 and gamma_k.dtype == torch.float32
    a.eps = eps
    a.rank, a.world = rank, world
    for p in range(world):
        a.head_splits[p] = head_splits[p]
        a.win_q[p], a.win_k[p], a.win_v[p], a.peer_ctrl[p] = win_q[p], win_k[p], win_v[p], ctrl[p]
    a.flags, a.timeout_ms, a.ctas = flags, timeout_ms, ctas
    a.win_bytes = win_bytes
    a.err = error_word(x.device).data_ptr()
    ck.check(ck.lib().fu_qkv_rope_scatter(C.byref(a), ck.stream_ptr()))


def qkv_reference(x: torch.Tensor, w: torch.Tensor, rope: torch.Tensor, gamma_q: torch.Tensor,
                  gamma_k: torch.Tensor, heads: int, eps: float = 1e-6):
    """fp32 PyTorch statement: matmul -> per-head RMSNorm (q, k) -> RoPE (q, k). Returns q, k, v
    of shape (b*s, heads, 128) for the local rows (before any exchange)."""
    from .rope import apply_rope_reference

    y = x.float() @ w.float().t()
    q, k, v = (t.reshape(x.shape[0], heads, HEAD_DIM) for t in y.chunk(3, dim=1))

    def norm(t, g):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * g.float()

    s_local = rope.shape[0]
    b = x.shape[0] // s_local

    def rot(t):
        t = t.reshape(b, s_local, heads, HEAD_DIM)
        return apply_rope_reference(t, rope).reshape(-1, heads, HEAD_DIM)

    return rot(norm(q, gamma_q)), rot(norm(k, gamma_k)), v


def qk_norm_rope_bwd(dq, dk, y_save, dy, rope, gamma_q, gamma_k, dgamma_q, dgamma_k, *, heads: int, s_local: int,
                     eps: float = 1e-6) -> None:
    """Backward of per-head RMSNorm -> RoPE for q and k (csrc/kernels/elementwise.cu). ``dq``/``dk``:
    (m, heads*128) bf16 dense; ``y_save``: (m, 2*heads*128) pre-norm projections; ``dy`` receives
    the q part at column 0 and the k part at column heads*128; ``dgamma_*`` fp32[128] accumulate."""
    m = dq.shape[0]
    assert dq.is_contiguous() and dk.is_contiguous() and dq.dtype == torch.bfloat16
    assert y_save.stride(1) == 1 and dy.stride(1) == 1
    a = ck.FuNormRopeBwdArgs()
    a.dq, a.dk, a.y, a.dy = dq.data_ptr(), dk.data_ptr(), y_save.data_ptr(), dy.data_ptr()
    gq, gk = gamma_q.detach().float().contiguous(), gamma_k.detach().float().contiguous()
    a.rope, a.gamma_q, a.gamma_k = rope.data_ptr(), gq.data_ptr(), gk.data_ptr()
    a.dgamma_q, a.dgamma_k = dgamma_q.data_ptr(), dgamma_k.data_ptr()
    a.m, a.s_local, a.ld_y, a.ld_dy = m, s_local, y_save.stride(0), dy.stride(0)
    a.heads, a.eps = heads, eps
    ck.check(ck.lib().fu_qk_norm_rope_bwd(C.byref(a), ck.stream_ptr()))


def pull_qkv_grads_raw(dy: torch.Tensor, y_save: torch.Tensor, rope: torch.Tensor, gamma_q: torch.Tensor,
                       gamma_k: torch.Tensor, dgamma_q: torch.Tensor, dgamma_k: torch.Tensor, *, heads: int,
                       s_local: int, seq_off: int, s_total: int, head_splits: list[int], rank: int,
                       peer_dq: list[int], peer_dk: list[int], peer_dv: list[int], ctrl: list[int], src_bytes: int,
                       eps: float = 1e-6, flags: int = 0, timeout_ms: int = 10000) -> None:
    """The exchange that brings dq, dk, dv home fused with the backward of RMSNorm -> RoPE
    (csrc/kernels/elementwise.cu:fu_pull_qkv_grads). ``peer_d*`` are the addresses of every rank's
    (b, s_total, head_splits[p], 128) bf16 gradient buffers, ``src_bytes`` the bytes behind each;
    ``dy`` (m, 3*heads*128) receives d(projection) for q | k | v; ``dgamma_*`` fp32[128] accumulate."""
    m = dy.shape[0]
    assert dy.dtype == torch.bfloat16 and dy.shape[1] == 3 * heads * HEAD_DIM and dy.stride(1) == 1
    assert y_save.dtype == torch.bfloat16 and y_save.shape == (m, 2 * heads * HEAD_DIM) and y_save.stride(1) == 1
    assert rope.dtype == torch.float32 and rope.shape == (s_local, HEAD_DIM // 2, 2) and rope.is_contiguous()
    for t in (gamma_q, gamma_k, dgamma_q, dgamma_k):
        assert t.dtype == torch.float32 and t.numel() == HEAD_DIM and t.is_contiguous()
    a = ck.FuPullGradsArgs()
    world = len(head_splits)
    for p in range(world):
        a.peer_dq[p], a.peer_dk[p], a.peer_dv[p], a.peer_ctrl[p] = peer_dq[p], peer_dk[p], peer_dv[p], ctrl[p]
        a.head_splits[p] = head_splits[p]
    a.src_bytes = src_bytes
    a.y, a.dy, a.rope = y_save.data_ptr(), dy.data_ptr(), rope.data_ptr()
    a.gamma_q, a.gamma_k = gamma_q.data_ptr(), gamma_k.data_ptr()
    a.dgamma_q, a.dgamma_k = dgamma_q.data_ptr(), dgamma_k.data_ptr()
    a.m, a.s_local, a.seq_off, a.s_total = m, s_local, seq_off, s_total
    a.ld_y, a.ld_dy = y_save.stride(0), dy.stride(0)
    a.heads, a.rank, a.world = heads, rank, world
    a.flags, a.timeout_ms, a.eps = flags, timeout_ms, eps
    ck.check(ck.lib().fu_pull_qkv_grads(C.byref(a), ck.stream_ptr()))
