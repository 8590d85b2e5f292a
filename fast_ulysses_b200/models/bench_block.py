"""Benchmark body for the sequence-parallel Wan2.1-14B-shaped attention block (forward+backward),
called by the repository's bench.py with its timing helper."""

from __future__ import annotations

import torch

from ..ops import gemm
from .attention import UlyssesSelfAttention

GRID, HIDDEN, HEADS = (21, 45, 80), 5120, 40


def bench_attention_block(group, world: int, rank: int, time_steps, flush, steps: int = 5, warmup: int = 3) -> dict:
    torch.manual_seed(1234)
    attn = UlyssesSelfAttention(group, HIDDEN, HEADS, grid=GRID)
    s_local = attn.s_local
    x = torch.randn(1, s_local, HIDDEN, device=group.device).bfloat16().requires_grad_()
    dy = torch.randn(1, s_local, HIDDEN, device=group.device).bfloat16()

    def fwd():
        with torch.no_grad():
            attn(x)

    def step():
        x.grad = None
        for p in attn.parameters():
            p.grad = None
        attn(x).backward(dy)

    out = {"config": {"hidden": HIDDEN, "heads": HEADS, "tokens": GRID[0] * GRID[1] * GRID[2],
                      "per_rank_x": [1, s_local, HIDDEN], "kernels": "fused qkv+norm+rope+scatter, tcgen05 fmha, "
                      "pull+outproj; backward: scatter-epilogue dgrad, tcgen05 fmha bwd, fused pull of dq/dk/dv + "
                      "norm/rope backward, tcgen05 dgrad/wgrad"}}
    # one step, then look at the error words before anything is looped: a kernel that gives up on an
    # internal wait takes seconds per launch, and a timing loop would multiply that
    step()
    gemm.check_errors()
    group.check()
    out["fwd_ms"] = time_steps(fwd, steps, warmup, world, flush)
    out["fwd_bwd_ms"] = time_steps(step, steps, warmup, world, flush)
    gemm.check_errors()
    group.check()
    return out
