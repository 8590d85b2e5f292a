"""A Wan2.1-14B-shaped DiT block stack (self-attention only) on the fused sequence-parallel kernels.

Block: x + Attn(LN(x)); x + FFN(LN(x)) with FFN = Linear(5120 -> 13824) -> GELU(tanh) ->
Linear(13824 -> 5120). Every contraction runs on the tcgen05 GEMM and everything between the
contractions lives in an epilogue: GELU (and, backward, its derivative), both residual adds and
the biases; LayerNorm is one kernel forward and one backward. No eager PyTorch elementwise kernel
runs inside a block. ``reference_forward`` is the same stack without sequence parallelism on one
device, the oracle for the multi-GPU tests.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.gemm import feed_forward
from ..ops.norm import layer_norm
from .attention import UlyssesSelfAttention, reference_attention


class DiTBlock(nn.Module):
    def __init__(self, group, hidden=5120, heads=40, ffn=13824, **attn_kw):
        super().__init__()
        dev = group.device
        self.hidden = hidden
        self.attn = UlyssesSelfAttention(group, hidden, heads, **attn_kw)
        self.w1 = nn.Parameter(torch.randn(ffn, hidden, device=dev).mul_(0.02).bfloat16())
        self.b1 = nn.Parameter(torch.zeros(ffn, device=dev).bfloat16())
        self.w2 = nn.Parameter(torch.randn(hidden, ffn, device=dev).mul_(0.02).bfloat16())
        self.b2 = nn.Parameter(torch.zeros(hidden, device=dev).bfloat16())

    def forward(self, x):
        x = self.attn(layer_norm(x), residual=x)  # x + Attn(LN(x)): the add is the out-projection's epilogue
        return feed_forward(layer_norm(x), self.w1, self.b1, self.w2, self.b2, residual=x)


class DiTStack(nn.Module):
    """``depth`` blocks over a sequence sharded across ``group``. Weight gradients are partial
    sums over this rank's sequence shard: call ``allreduce_grads()`` after backward."""

    def __init__(self, group, depth=4, hidden=5120, heads=40, ffn=13824, **attn_kw):
        super().__init__()
        self.group = group
        self.blocks = nn.ModuleList([DiTBlock(group, hidden, heads, ffn, **attn_kw) for _ in range(depth)])

    def forward(self, x):
        for blk in self.blocks:
            x = blk(x)
        return x

    def allreduce_grads(self):
        import torch.distributed as dist

        if self.group.world_size == 1:
            return
        for p in self.parameters():
            if p.grad is not None:
                dist.all_reduce(p.grad, group=self.group.pg)


def reference_forward(stack: DiTStack, x_full: torch.Tensor, compute=torch.float32) -> torch.Tensor:
    """The same blocks applied to the FULL sequence on one device, plain PyTorch."""
    x = x_full.to(compute)
    for blk in stack.blocks:
        a = blk.attn
        hdn = blk.hidden
        x = x + reference_attention(F.layer_norm(x, (hdn,), eps=1e-6), a.w_qkv, a.gamma_q, a.gamma_k, a.w_o, a.b_o,
                                    a.heads, a.grid, a.eps, compute)
        h = F.gelu(F.linear(F.layer_norm(x, (hdn,), eps=1e-6), blk.w1.to(compute), blk.b1.to(compute)),
                   approximate="tanh")
        x = x + F.linear(h, blk.w2.to(compute), blk.b2.to(compute))
    return x
