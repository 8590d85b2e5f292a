"""Sequence-parallel self-attention for video DiT blocks, built from the fused sm_100a kernels.

Forward (three kernels, no separate exchange, no permute, no staging copy):
  1. ``fu_qkv_rope_scatter``  x W_qkv^T -> per-head RMSNorm -> 3D RoPE -> every head-row stored
     straight into the owning rank's q/k/v window (mode 0 of the all-to-all is the store address)
  2. ``fu_fmha_fwd``          tcgen05 flash attention reading q/k/v from the window, writing the
     attention output into a symmetric buffer
  3. ``fu_pull_outproj``      the output projection pulls its A operand from the peers' attention
     outputs tile by tile (mode 1 of the all-to-all is the load address)
Backward mirrors it: the gradient of the attention output is scattered to the head owners from
the epilogue of the dgrad GEMM (same kernel as 1 without norm/RoPE), tcgen05 flash attention
backward, one ``all_to_all_4d`` (mode 1) brings dq/dk/dv home, a fused RMSNorm/RoPE backward
feeds the dgrad/wgrad GEMMs.

The reference ships no model code; its example (examples/dit_attention.py:21-63) wraps nn.Linear
and torch SDPA around two all_to_all_4d calls. ``reference_attention`` below is that composition,
used as the oracle.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import _ckernels as ck
from ..ops import attention as fa
from ..ops import gemm, outproj, qkv
from ..ops.rope import apply_rope_reference, rope_table

HEAD_DIM = 128


class SymmBuffer:
    """A caller-owned symmetric byte buffer plus its address on every rank."""

    def __init__(self, group, nbytes: int):
        nbytes = (nbytes + 255) // 256 * 256
        self.tensor = group._handle.symm_alloc(nbytes)
        ptrs = group._handle.symm_ptrs(self.tensor)
        w = group.world_size
        self.base, self.ctrl = list(ptrs[:w]), list(ptrs[w:])
        self.nbytes = nbytes

    def view(self, offset: int, shape, dtype=torch.bfloat16) -> torch.Tensor:
        n = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
        return self.tensor[offset:offset + n].view(dtype).view(*shape)


class _SPAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_qkv, gamma_q, gamma_k, w_o, b_o, mod):
        b, s_local, hidden = x.shape
        m = b * s_local
        x2 = x.reshape(m, hidden)
        if x2.stride(1) != 1 or x2.stride(0) % 8:
            x2 = x2.contiguous()
        N = mod.heads
        need_grad = any(ctx.needs_input_grad[:6])
        # q, k, v and the attention output live in the module's symmetric buffers, not in tensors
        # saved for backward: a second forward overwrites them. Number the forwards so that a
        # backward which would read another call's activations refuses instead.
        mod._forward_count += 1
        y_save = torch.empty(m, 2 * N * HEAD_DIM, dtype=torch.bfloat16, device=x.device) if need_grad else None
        mod._launch_scatter(x2, w_qkv, mod.qkv_win, 3, 2, gamma_q, gamma_k, y_save)
        q, k, v = mod.q_view, mod.k_view, mod.v_view
        _, lse = fa.fmha_fwd(q, k, v, out=mod.o_view)
        gather = torch.empty(m, N * HEAD_DIM, dtype=torch.bfloat16, device=x.device)
        out = torch.empty(m, hidden, dtype=torch.bfloat16, device=x.device)
        ready = mod._ready_flags(m)
        outproj.pull_outproj_raw(w_o, out, gather, ready, s_local=s_local, seq_off=mod.seq_off, s_total=mod.s_total,
                                 head_splits=mod.head_splits, rank=mod.rank, peer_o=mod.o_buf.base, ctrl=mod.o_buf.ctrl,
                                 o_bytes=mod._region,
                                 bias=mod._f32("b_o", b_o) if b_o is not None else None, timeout_ms=mod.timeout_ms)
        if need_grad:
            ctx.save_for_backward(x2, w_qkv, gamma_q, gamma_k, w_o, y_save, gather, lse)
            ctx.mod = mod
            ctx.forward_id = mod._forward_count
            ctx.has_bias = b_o is not None
            ctx.x_shape = x.shape
        return out.view(b, s_local, hidden)

    @staticmethod
    def backward(ctx, dy):
        x2, w_qkv, gamma_q, gamma_k, w_o, y_save, gather, lse = ctx.saved_tensors
        mod = ctx.mod
        if ctx.forward_id != mod._forward_count:
            raise RuntimeError(
                "UlyssesSelfAttention: forward ran again on this module before this backward; q, k, v and the "
                "attention output live in the module's symmetric buffers and now belong to the later call "
                f"(this backward is for forward #{ctx.forward_id}, the buffers hold #{mod._forward_count}). Run "
                "backward before the next forward (gradient accumulation: forward, backward, forward, backward), "
                "use one module per activation that must stay alive, or recompute the forward.")
        b, s_local, hidden = ctx.x_shape
        m, N = b * s_local, mod.heads
        dy2 = dy.reshape(m, hidden)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        db_o = dy2.sum(0, dtype=torch.float32).to(dy.dtype) if ctx.has_bias else None
        # dW_o[n, k] = sum_m dy[m, n] A[m, k]
        dw_o = gemm.gemm_bf16(dy2, gather, a_km=True, b_kn=True)
        # dA = dy W_o, scattered to the head owners from the GEMM epilogue (mode-0 direction)
        mod._launch_scatter(dy2, w_o.t().contiguous(), mod.do_win, 1, 0, None, None, None)
        dqkv = torch.empty(3, b, mod.s_total, mod.n_local, HEAD_DIM, dtype=torch.bfloat16, device=dy.device)
        fa.fmha_bwd(mod.q_view, mod.k_view, mod.v_view, mod.o_view, lse, mod.do_view,
                    out=(dqkv[0], dqkv[1], dqkv[2]))
        # dq, dk, dv go home in one exchange (mode 1), the three tensors folded into the batch axis
        back = mod.group.all_to_all_4d(dqkv.view(3 * b, mod.s_total, mod.n_local, HEAD_DIM), mode=1,
                                       seq_splits=mod.seq_splits, head_splits=mod.head_splits)
        back = back.view(3, m, N * HEAD_DIM)
        dyqkv = torch.empty(m, 3 * N * HEAD_DIM, dtype=torch.bfloat16, device=dy.device)
        dgq = torch.zeros(HEAD_DIM, dtype=torch.float32, device=dy.device)
        dgk = torch.zeros(HEAD_DIM, dtype=torch.float32, device=dy.device)
        qkv.qk_norm_rope_bwd(back[0], back[1], y_save, dyqkv, mod.rope, gamma_q, gamma_k, dgq, dgk, heads=N,
                             s_local=s_local, eps=mod.eps)
        dyqkv[:, 2 * N * HEAD_DIM:].copy_(back[2])
        dx = gemm.gemm_bf16(dyqkv, w_qkv, b_kn=True).view(b, s_local, hidden)
        dw_qkv = gemm.gemm_bf16(dyqkv, x2, a_km=True, b_kn=True)
        return dx, dw_qkv, dgq.to(gamma_q.dtype), dgk.to(gamma_k.dtype), dw_o, db_o, None


class UlyssesSelfAttention(nn.Module):
    """Self-attention over a sequence sharded across ``group`` (Ulysses), Wan2.1-style: fused QKV
    projection, per-head RMSNorm on q and k, 3D RoPE, non-causal attention, output projection.

    Construction is collective (it allocates symmetric buffers). ``seq_splits`` / ``head_splits``
    give every rank's shard (default: even). Input ``(b, s_local, hidden)`` bf16.
    """

    def __init__(self, group, hidden: int = 5120, heads: int = 40, *, grid=(21, 45, 80), batch: int = 1,
                 seq_splits: list[int] | None = None, head_splits: list[int] | None = None, eps: float = 1e-6,
                 out_bias: bool = True, timeout_ms: int = 10000):
        super().__init__()
        self.group, self.hidden, self.heads, self.grid, self.eps = group, hidden, heads, grid, eps
        self.rank, self.world = group.rank, group.world_size
        total = grid[0] * grid[1] * grid[2]
        if seq_splits is None:
            assert total % self.world == 0, "pass seq_splits for a sequence that does not divide"
            seq_splits = [total // self.world] * self.world
        if head_splits is None:
            assert heads % self.world == 0, "pass head_splits for a head count that does not divide"
            head_splits = [heads // self.world] * self.world
        assert sum(seq_splits) == total and sum(head_splits) == heads
        self.seq_splits, self.head_splits = list(seq_splits), list(head_splits)
        self.s_total, self.s_local = total, seq_splits[self.rank]
        self.seq_off = sum(seq_splits[: self.rank])
        self.n_local = head_splits[self.rank]
        self.batch, self.timeout_ms = batch, timeout_ms
        dev = group.device

        self.w_qkv = nn.Parameter(torch.randn(3 * heads * HEAD_DIM, hidden, device=dev).mul_(0.02).bfloat16())
        self.w_o = nn.Parameter(torch.randn(hidden, heads * HEAD_DIM, device=dev).mul_(0.02).bfloat16())
        self.b_o = nn.Parameter(torch.zeros(hidden, device=dev).bfloat16()) if out_bias else None
        self.gamma_q = nn.Parameter(torch.ones(HEAD_DIM, device=dev))
        self.gamma_k = nn.Parameter(torch.ones(HEAD_DIM, device=dev))
        self.register_buffer("rope", rope_table(torch.arange(self.seq_off, self.seq_off + self.s_local, device=dev),
                                                grid=grid), persistent=False)

        # Symmetric buffers. Every rank sizes them for the LARGEST head shard, so that offsets agree.
        region = batch * total * max(head_splits) * HEAD_DIM * 2
        region = (region + 255) // 256 * 256
        self._region = region
        self.qkv_win = SymmBuffer(group, 3 * region)
        self.o_buf = SymmBuffer(group, region)
        self.do_win = SymmBuffer(group, region)
        shape = (batch, total, self.n_local, HEAD_DIM)
        self.q_view = self.qkv_win.view(0, shape)
        self.k_view = self.qkv_win.view(region, shape)
        self.v_view = self.qkv_win.view(2 * region, shape)
        self.o_view = self.o_buf.view(0, shape)
        self.do_view = self.do_win.view(0, shape)
        self._ready = None
        self._forward_count = 0
        self._f32_cache: dict[str, tuple[int, torch.Tensor]] = {}

    def _f32(self, name: str, param: torch.Tensor) -> torch.Tensor:
        """fp32 copy of a small parameter, remade only when the parameter has changed in place."""
        hit = self._f32_cache.get(name)
        key = (param._version, param.data_ptr())
        if hit is None or hit[0] != key:
            hit = (key, param.detach().float().contiguous())
            self._f32_cache[name] = hit
        return hit[1]

    def _ready_flags(self, m: int) -> torch.Tensor:
        n = ((m + 127) // 128) * self.world
        if self._ready is None or self._ready.numel() < n:
            self._ready = torch.zeros(n, dtype=torch.int32, device=self.group.device)
        return self._ready

    def _launch_scatter(self, x2, w, win: SymmBuffer, n_types, n_normed, gamma_q, gamma_k, y_save):
        import ctypes as C

        a = ck.FuQkvArgs()
        a.x, a.w = x2.data_ptr(), w.data_ptr()
        a.m, a.k, a.ldx, a.ldw = x2.shape[0], x2.shape[1], x2.stride(0), w.stride(0)
        a.heads = self.heads
        a.s_local, a.seq_off, a.s_total = self.s_local, self.seq_off, self.s_total
        a.eps = self.eps
        a.rank, a.world = self.rank, self.world
        if n_normed:
            gq32, gk32 = self._f32("gamma_q", gamma_q), self._f32("gamma_k", gamma_k)
            a.rope, a.gamma_q, a.gamma_k = self.rope.data_ptr(), gq32.data_ptr(), gk32.data_ptr()
        for p in range(self.world):
            a.head_splits[p] = self.head_splits[p]
            a.win_q[p] = win.base[p]
            a.win_k[p] = win.base[p] + self._region
            a.win_v[p] = win.base[p] + 2 * self._region
            a.peer_ctrl[p] = win.ctrl[p]
        a.timeout_ms = self.timeout_ms
        a.err = gemm.error_word(x2.device).data_ptr()
        a.n_types, a.n_normed = n_types, n_normed
        a.win_bytes = self._region
        if y_save is not None:
            a.y_save, a.ld_y = y_save.data_ptr(), y_save.stride(0)
        assert w.shape[0] == n_types * self.heads * HEAD_DIM and x2.dtype == torch.bfloat16
        ck.check(ck.lib().fu_qkv_rope_scatter(C.byref(a), ck.stream_ptr()))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        assert x.shape[0] == self.batch and x.shape[1] == self.s_local and x.dtype == torch.bfloat16, x.shape
        return _SPAttention.apply(x, self.w_qkv, self.gamma_q, self.gamma_k, self.w_o, self.b_o, self)


def reference_attention(x_full, w_qkv, gamma_q, gamma_k, w_o, b_o, heads, grid, eps=1e-6, compute=torch.float32):
    """The same block without sequence parallelism, in plain PyTorch on the FULL sequence
    (b, S, hidden): linear -> per-head RMSNorm -> RoPE -> SDPA -> linear."""
    b, S, hidden = x_full.shape
    xf = x_full.to(compute)
    y = xf @ w_qkv.to(compute).t()
    q, k, v = (t.reshape(b, S, heads, HEAD_DIM) for t in y.chunk(3, dim=-1))

    def norm(t, g):
        return t * torch.rsqrt(t.float().pow(2).mean(-1, keepdim=True) + eps).to(t.dtype) * g.to(t.dtype)

    table = rope_table(torch.arange(S, device=x_full.device), grid=grid)
    q = apply_rope_reference(norm(q, gamma_q), table).to(compute)
    k = apply_rope_reference(norm(k, gamma_k), table).to(compute)
    o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    o = o.transpose(1, 2).reshape(b, S, heads * HEAD_DIM)
    out = o @ w_o.to(compute).t()
    return out + b_o.to(compute) if b_o is not None else out
