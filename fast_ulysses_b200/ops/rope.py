"""3D rotary position tables for video DiT attention (Wan2.1 layout).

A token's position is its (frame, row, column) in a ``grid = (t, h, w)`` latent volume; the head
dimension is split ``(44, 42, 42)`` between the three axes, each part rotated pairwise
(elements ``2i, 2i+1``) with frequencies ``theta ** (-2i / part_dim)``.
"""

from __future__ import annotations

import torch


def rope_table(token_index: torch.Tensor, grid=(21, 45, 80), head_dim: int = 128, splits=(44, 42, 42),
               theta: float = 10000.0) -> torch.Tensor:
    """``(len(token_index), head_dim // 2, 2)`` float32 table of (cos, sin) per rotated pair.

    ``token_index`` holds GLOBAL token numbers (row-major over ``grid``), so a sequence shard
    passes ``arange(seq_off, seq_off + s_local)``."""
    assert sum(splits) == head_dim and all(s % 2 == 0 for s in splits)
    t, h, w = grid
    idx = token_index.to(torch.int64)
    pos = (idx // (h * w), (idx // w) % h, idx % w)
    parts = []
    for p, dim in zip(pos, splits):
        freqs = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64, device=idx.device) / dim))
        parts.append(p.to(torch.float64)[:, None] * freqs[None, :])
    ang = torch.cat(parts, dim=1)  # (n, head_dim // 2)
    return torch.stack((ang.cos(), ang.sin()), dim=-1).to(torch.float32).contiguous()


def apply_rope_reference(x: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Plain PyTorch statement: ``x`` is (..., s, heads, head_dim), ``table`` is (s, head_dim/2, 2)."""
    xf = x.float().reshape(*x.shape[:-1], -1, 2)
    cos = table[:, None, :, 0]
    sin = table[:, None, :, 1]
    x0, x1 = xf[..., 0], xf[..., 1]
    return torch.stack((x0 * cos - x1 * sin, x0 * sin + x1 * cos), dim=-1).reshape(x.shape)
