"""Sequence-parallel self-attention for video DiT blocks, built from the fused sm_100a kernels.

Forward (three kernels, no separate exchange, no permute, no staging copy):
  1. ``fu_qkv_rope_scatter``  x W_qkv^T -> per-head RMSNorm -> 3D RoPE -> every head-row stored
     straight into the owning rank's q/k/v window (mode 0 of the all-to-all is the store address)
  2. ``fu_fmha_fwd``          tcgen05 flash attention reading q/k/v from the window, writing the
     attention output into a symmetric buffer
  3. ``fu_pull_outproj``      the output projection pulls its A operand from the peers' attention
     outputs tile by tile (mode 1 of the all-to-all is the load address)
Backward mirrors it: the gradient of the attention output is scattered to the head owners from
the epilogue of the dgrad GEMM (same kernel as 1 without norm/RoPE, reading W_o as stored),
tcgen05 flash attention backward writes dq/dk/dv into a symmetric buffer, and ONE kernel
(``fu_pull_qkv_grads``) pulls them home from the head owners over NVLink while undoing RoPE and
RMSNorm on the way and writes the operand of the dgrad/wgrad GEMMs: no stand-alone exchange, no
separate norm/RoPE backward, no slice copy, no transposed weight.

The reference ships no model code; its example (examples/dit_attention.py:21-63) wraps nn.Linear
and torch SDPA around two all_to_all_4d calls. ``reference_attention`` below is that composition,
used as the oracle.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
from torch.cuda import nvtx

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
    def forward(ctx, x, w_qkv, gamma_q, gamma_k, w_o, b_o, residual, mod):
        b, s_local, hidden = x.shape
        m = b * s_local
        x2 = x.reshape(m, hidden)
        if x2.stride(1) != 1 or x2.stride(0) % 8:
            x2 = x2.contiguous()
        N = mod.heads
        need_grad = any(ctx.needs_input_grad[:7])
        # q, k, v and the attention output live in the module's symmetric buffers, not in tensors
        # saved for backward: a second forward overwrites them. Number the forwards so that a
        # backward which would read another call's activations refuses instead.
        mod._forward_count += 1
        y_save = torch.empty(m, 2 * N * HEAD_DIM, dtype=torch.bfloat16, device=x.device) if need_grad else None
        with nvtx.range("fast_ulysses_b200::qkv_norm_rope_scatter"):
            mod._launch_scatter(x2, w_qkv, mod.qkv_win, 3, 2, gamma_q, gamma_k, y_save)
        q, k, v = mod.q_view, mod.k_view, mod.v_view
        with nvtx.range("fast_ulysses_b200::fmha_fwd"):
            _, lse = fa.fmha_fwd(q, k, v, out=mod.o_view)
        gather = torch.empty(m, N * HEAD_DIM, dtype=torch.bfloat16, device=x.device)
        out = torch.empty(m, hidden, dtype=torch.bfloat16, device=x.device)
        ready = mod._ready_flags(m)
        res2 = None
        if residual is not None:  # added in the out-projection's epilogue
            res2 = residual.reshape(m, hidden)
            if not res2.is_contiguous():
                res2 = res2.contiguous()
        with nvtx.range("fast_ulysses_b200::pull_outproj"):
            outproj.pull_outproj_raw(w_o, out, gather, ready, s_local=s_local, seq_off=mod.seq_off,
                                     s_total=mod.s_total, head_splits=mod.head_splits, rank=mod.rank,
                                     peer_o=mod.o_buf.base, ctrl=mod.o_buf.ctrl, o_bytes=mod._region,
                                     bias=mod._f32("b_o", b_o) if b_o is not None else None,
                                     residual=res2, timeout_ms=mod.timeout_ms, ctas=mod._fused_ctas())
        if need_grad:
            ctx.save_for_backward(x2, w_qkv, gamma_q, gamma_k, w_o, y_save, gather, lse)
            ctx.mod = mod
            ctx.forward_id = mod._forward_count
            ctx.has_bias = b_o is not None
            ctx.has_residual = residual is not None
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
        # dA = dy W_o, scattered to the head owners from the GEMM epilogue (mode-0 direction); W_o is
        # (hidden, heads * 128) = (contraction, output) as stored, so nothing is transposed
        with nvtx.range("fast_ulysses_b200::dout_scatter"):
            mod._launch_scatter(dy2, w_o, mod.do_win, 1, 0, None, None, None, w_kn=True)
        with nvtx.range("fast_ulysses_b200::fmha_bwd"):
            fa.fmha_bwd(mod.q_view, mod.k_view, mod.v_view, mod.o_view, lse, mod.do_view,
                        out=(mod.dq_view, mod.dk_view, mod.dv_view))
        # dq, dk, dv come home inside the kernel that undoes RoPE and RMSNorm (mode-1 direction)
        dyqkv = torch.empty(m, 3 * N * HEAD_DIM, dtype=torch.bfloat16, device=dy.device)
        dgq = torch.zeros(HEAD_DIM, dtype=torch.float32, device=dy.device)
        dgk = torch.zeros(HEAD_DIM, dtype=torch.float32, device=dy.device)
        R = mod._region
        with nvtx.range("fast_ulysses_b200::pull_qkv_grads"):
            qkv.pull_qkv_grads_raw(dyqkv, y_save, mod.rope, mod._f32("gamma_q", gamma_q), mod._f32("gamma_k", gamma_k),
                                   dgq, dgk, heads=N, s_local=s_local, seq_off=mod.seq_off, s_total=mod.s_total,
                                   head_splits=mod.head_splits, rank=mod.rank, peer_dq=mod.dqkv_buf.base,
                                   peer_dk=[p + R for p in mod.dqkv_buf.base],
                                   peer_dv=[p + 2 * R for p in mod.dqkv_buf.base], ctrl=mod.dqkv_buf.ctrl,
                                   src_bytes=R, eps=mod.eps, timeout_ms=mod.timeout_ms)
        dx = gemm.gemm_bf16(dyqkv, w_qkv, b_kn=True).view(b, s_local, hidden)
        dw_qkv = gemm.gemm_bf16(dyqkv, x2, a_km=True, b_kn=True)
        return (dx, dw_qkv, dgq.to(gamma_q.dtype), dgk.to(gamma_k.dtype), dw_o, db_o,
                dy if ctx.has_residual else None, None)


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
        self.dqkv_buf = SymmBuffer(group, 3 * region)  # dq | dk | dv of this rank's heads, pulled by the token owners
        shape = (batch, total, self.n_local, HEAD_DIM)
        self.q_view = self.qkv_win.view(0, shape)
        self.k_view = self.qkv_win.view(region, shape)
        self.v_view = self.qkv_win.view(2 * region, shape)
        self.o_view = self.o_buf.view(0, shape)
        self.do_view = self.do_win.view(0, shape)
        self.dq_view = self.dqkv_buf.view(0, shape)
        self.dk_view = self.dqkv_buf.view(region, shape)
        self.dv_view = self.dqkv_buf.view(2 * region, shape)
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

    def _fused_ctas(self) -> int:
        """How many CTAs a fused GEMM kernel of this block may take right now (0 = the whole device).

        The fused kernels are persistent, one CTA per SM, and their CTAs wait on peers; an
        asynchronous exchange of the same group is a kernel of the same kind on another stream.
        If one held every SM on this rank while the other could not start here, and the opposite
        happened on a peer, each would wait for a kernel that cannot run. So while the group's comm
        stream has work queued, a fused kernel leaves the SMs an asynchronous exchange takes (a
        third of the device) free; with the comm stream idle it takes everything. All ranks issue
        the same calls in the same order, so a rank that sees its comm stream idle has an exchange
        that every peer has already been able to start."""
        comm = getattr(self.group, "_comm_stream", None)
        if self.world == 1 or comm is None or comm.query():
            return 0
        sms = torch.cuda.get_device_properties(self.group.device).multi_processor_count
        return sms - sms // 3

    def _ready_flags(self, m: int) -> torch.Tensor:
        n = ((m + 127) // 128) * self.world
        if self._ready is None or self._ready.numel() < n:
            self._ready = torch.zeros(n, dtype=torch.int32, device=self.group.device)
        return self._ready

    def _launch_scatter(self, x2, w, win: SymmBuffer, n_types, n_normed, gamma_q, gamma_k, y_save, w_kn=False):
        """``w_kn``: the weight is (contraction, output) as stored instead of (output, contraction)."""
        import ctypes as C

        a = ck.FuQkvArgs()
        a.x, a.w = x2.data_ptr(), w.data_ptr()
        a.m, a.k, a.ldx, a.ldw = x2.shape[0], x2.shape[1], x2.stride(0), w.stride(0)
        a.flags = ck.FU_QKV_W_KN if w_kn else 0
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
        a.ctas = self._fused_ctas()
        a.err = gemm.error_word(x2.device).data_ptr()
        a.n_types, a.n_normed = n_types, n_normed
        a.win_bytes = self._region
        if y_save is not None:
            a.y_save, a.ld_y = y_save.data_ptr(), y_save.stride(0)
        assert w.shape[1 if w_kn else 0] == n_types * self.heads * HEAD_DIM and x2.dtype == torch.bfloat16
        assert w.shape[0 if w_kn else 1] == x2.shape[1] and w.stride(1) == 1
        ck.check(ck.lib().fu_qkv_rope_scatter(C.byref(a), ck.stream_ptr()))

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """``residual`` (same shape as the result) is added in the output projection's epilogue."""
        assert x.shape[0] == self.batch and x.shape[1] == self.s_local and x.dtype == torch.bfloat16, x.shape
        assert residual is None or (residual.shape == x.shape and residual.dtype == torch.bfloat16)
        return _SPAttention.apply(x, self.w_qkv, self.gamma_q, self.gamma_k, self.w_o, self.b_o, residual, self)


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
