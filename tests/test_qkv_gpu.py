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


def test_pull_qkv_grads_matches_exchange_then_norm_rope_backward():
    """The fused backward entry (pull dq, dk, dv from the head owners, undo RoPE and RMSNorm on the
    way) against the unfused statement: gather by slicing, then the stand-alone backward kernel.
    Three emulated ranks with uneven shards on one device, handshakes off."""
    torch.manual_seed(21)
    seq, head_splits, grid, b = [40, 17, 63], [2, 1, 3], (4, 6, 10), 2
    world, heads, S = len(seq), sum(head_splits), sum(seq)
    region = b * S * max(head_splits) * 256
    # every rank's dq | dk | dv for its own heads over the whole sequence
    bufs = [torch.zeros(3 * region + ck.FU_CTRL_BYTES, dtype=torch.uint8, device="cuda") for _ in range(world)]
    full = [torch.randn(b, S, heads, 128, device="cuda").bfloat16() for _ in range(3)]  # global dq, dk, dv
    h0 = 0
    for p, hp in enumerate(head_splits):
        for t in range(3):
            bufs[p][t * region: t * region + b * S * hp * 256].view(torch.bfloat16).view(b, S, hp, 128).copy_(
                full[t][:, :, h0:h0 + hp])
        h0 += hp
    gq = (1 + 0.1 * torch.randn(128, device="cuda")).float()
    gk = (1 + 0.1 * torch.randn(128, device="cuda")).float()
    s0 = 0
    for r in range(world):
        m = b * seq[r]
        y_save = torch.randn(m, 2 * heads * 128, device="cuda").bfloat16()
        rope = rope_table(torch.arange(s0, s0 + seq[r], device="cuda"), grid=grid)
        dy = torch.zeros(m, 3 * heads * 128, device="cuda", dtype=torch.bfloat16)
        dgq, dgk = torch.zeros(128, device="cuda"), torch.zeros(128, device="cuda")
        qkv.pull_qkv_grads_raw(dy, y_save, rope, gq, gk, dgq, dgk, heads=heads, s_local=seq[r], seq_off=s0, s_total=S,
                               head_splits=head_splits, rank=r, peer_dq=[t.data_ptr() for t in bufs],
                               peer_dk=[t.data_ptr() + region for t in bufs],
                               peer_dv=[t.data_ptr() + 2 * region for t in bufs],
                               ctrl=[t.data_ptr() + 3 * region for t in bufs], src_bytes=region,
                               flags=ck.FU_A2A_NO_HANDSHAKE)
        # unfused: this rank's rows of the global gradients, then the stand-alone kernel
        mine = [f[:, s0:s0 + seq[r]].reshape(m, heads * 128).contiguous() for f in full]
        want = torch.zeros_like(dy)
        wgq, wgk = torch.zeros(128, device="cuda"), torch.zeros(128, device="cuda")
        qkv.qk_norm_rope_bwd(mine[0], mine[1], y_save, want, rope, gq, gk, wgq, wgk, heads=heads, s_local=seq[r])
        want[:, 2 * heads * 128:].copy_(mine[2])
        torch.cuda.synchronize()
        assert torch.equal(dy, want), f"rank {r}: d(projection)"
        assert torch.allclose(dgq, wgq, rtol=1e-3, atol=1e-3) and torch.allclose(dgk, wgk, rtol=1e-3, atol=1e-3)
        s0 += seq[r]
