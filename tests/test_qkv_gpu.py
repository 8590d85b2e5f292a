"""The fused QKV + RMSNorm + RoPE + scatter kernel on one GPU: a single rank, and three emulated
ranks with uneven head shards (fake peer windows on one device, handshakes off, ranks run one
after another). Oracle: fp32 matmul -> RMSNorm -> RoPE -> the permutation, in plain PyTorch."""

import pytest
import torch

from fast_ulysses_b200.ops import _ckernels as ck
from fast_ulysses_b200.ops import gemm, qkv
from fast_ulysses_b200.ops.rope import rope_table

pytestmark = pytest.mark.gpu


def run_world(seq, head_splits, hidden, b=1, grid=(4, 6, 10)):
    world = len(seq)
    heads = sum(head_splits)
    S = sum(seq)
    assert S <= grid[0] * grid[1] * grid[2]
    torch.manual_seed(7)
    w = (torch.randn(3 * heads * 128, hidden, device="cuda") * 0.05).bfloat16()
    gq = (1 + 0.1 * torch.randn(128, device="cuda")).float()
    gk = (1 + 0.1 * torch.randn(128, device="cuda")).float()
    region = b * S * max(head_splits) * 128 * 2
    wins = [torch.zeros(3 * region + ck.FU_CTRL_BYTES, dtype=torch.uint8, device="cuda") for _ in range(world)]
    xs, refs = [], []
    s0 = 0
    for r in range(world):
        x = torch.randn(b * seq[r], hidden, device="cuda").bfloat16()
        rope = rope_table(torch.arange(s0, s0 + seq[r], device="cuda"), grid=grid)
        qkv.qkv_rope_scatter_raw(
            x, w, rope, gq, gk, heads=heads, s_local=seq[r], seq_off=s0, s_total=S, head_splits=head_splits, rank=r,
            win_q=[t.data_ptr() for t in wins], win_k=[t.data_ptr() + region for t in wins],
            win_v=[t.data_ptr() + 2 * region for t in wins], ctrl=[t.data_ptr() + 3 * region for t in wins],
            win_bytes=region, flags=ck.FU_A2A_NO_HANDSHAKE)
        refs.append(qkv.qkv_reference(x, w, rope, gq, gk, heads))
        xs.append(x)
        s0 += seq[r]
    torch.cuda.synchronize()
    gemm.check_errors()
    h0 = 0
    for p in range(world):
        hp = head_splits[p]
        for t, name in enumerate("qkv"):
            got = wins[p][t * region: t * region + b * S * hp * 256].view(torch.bfloat16).view(b, S, hp, 128)
            want = torch.cat([refs[r][t].view(b, seq[r], heads, 128)[:, :, h0:h0 + hp] for r in range(world)], dim=1)
            err = ((got.float() - want).norm() / want.norm()).item()
            assert err < 1e-2, f"rank {p} {name}: rel err {err}"
        h0 += hp


def test_single_rank():
    run_world([200], [4], 256)


def test_single_rank_batched_and_partial_tile():
    run_world([77], [6], 320, b=2)


def test_three_ranks_uneven_heads():
    run_world([100, 60, 80], [3, 2, 3], 256)


def test_wan_head_layout_14_13_13():
    run_world([40, 30, 50], [14, 13, 13], 128)
