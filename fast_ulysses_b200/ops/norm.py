"""LayerNorm without affine parameters as one kernel forward and one backward
(csrc/kernels/elementwise.cu: fu_layernorm_fwd / fu_layernorm_bwd): bf16 in and out, statistics in
fp32. The DiT blocks normalise with it so that no eager elementwise kernel runs between the GEMMs."""

from __future__ import annotations

import torch

from . import _ckernels as ck


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, eps):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
            x2 = x2.contiguous()
        rows, cols = x2.shape
        assert x.dtype == torch.bfloat16 and cols % 8 == 0, (x.dtype, cols)
        y = torch.empty(rows, cols, dtype=torch.bfloat16, device=x.device)
        stats = torch.empty(rows, 2, dtype=torch.float32, device=x.device)
        ck.check(ck.lib().fu_layernorm_fwd(x2.data_ptr(), y.data_ptr(), stats.data_ptr(), rows, cols, x2.stride(0), cols,
                                           eps, ck.stream_ptr()))
        ctx.save_for_backward(x2, stats)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, gy):
        x2, stats = ctx.saved_tensors
        rows, cols = x2.shape
        g2 = gy.reshape(rows, cols)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        xc = x2 if x2.is_contiguous() else x2.contiguous()
        dx = torch.empty(rows, cols, dtype=torch.bfloat16, device=gy.device)
        ck.check(ck.lib().fu_layernorm_bwd(g2.data_ptr(), xc.data_ptr(), stats.data_ptr(), dx.data_ptr(), rows, cols, cols,
                                           ck.stream_ptr()))
        return dx.view(ctx.shape), None


def layer_norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``(x - mean) / sqrt(var + eps)`` over the last axis of a bf16 tensor (no weight, no bias)."""
    return _LayerNorm.apply(x, eps)
