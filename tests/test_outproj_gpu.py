"""The fused pull + output projection on one GPU: emulated ranks (peer O buffers on one device,
handshakes off), uneven head and sequence shards. Oracle: fp32 permutation -> matmul."""

import pytest
import torch

from fast_ulysses_b200.ops import _ckernels as ck
from fast_ulysses_b200.ops import gemm, outproj

pytestmark = pytest.mark.gpu


def run_world(seq, head_splits, n_out, b=1, ctas=0):
    world, heads, S = len(seq), sum(head_splits), sum(seq)
    torch.manual_seed(11)
    # each rank's attention output: (b, S, heads_p, 128) + control block
    o_bufs = [torch.randn(b, S, hp, 128, device="cuda").bfloat16() for hp in head_splits]
    ctrls = [torch.zeros(ck.FU_CTRL_BYTES, dtype=torch.uint8, device="cuda") for _ in range(world)]
    w = (torch.randn(n_out, heads * 128, device="cuda") * 0.05).bfloat16()
    bias = torch.randn(n_out, device="cuda")
    full = torch.cat(o_bufs, dim=2)  # (b, S, heads, 128): what the gather must reproduce
    s0 = 0
    for r in range(world):
        m = b * seq[r]
        res = torch.randn(m, n_out, device="cuda").bfloat16()
        out = torch.empty(m, n_out, device="cuda", dtype=torch.bfloat16)
        gather = torch.zeros(m, heads * 128, device="cuda", dtype=torch.bfloat16)
        ready = torch.zeros(((m + 127) // 128) * world, dtype=torch.int32, device="cuda")
        outproj.pull_outproj_raw(w, out, gather, ready, s_local=seq[r], seq_off=s0, s_total=S,
                                 head_splits=head_splits, rank=r, peer_o=[t.data_ptr() for t in o_bufs],
                                 ctrl=[t.data_ptr() for t in ctrls], o_bytes=b * S * max(head_splits) * 256,
                                 bias=bias, residual=res,
                                 flags=ck.FU_A2A_NO_HANDSHAKE, ctas=ctas)
        torch.cuda.synchronize()
        gemm.check_errors()
        a_ref = full[:, s0:s0 + seq[r]].reshape(m, heads * 128)
        assert torch.equal(gather, a_ref), f"rank {r}: gathered operand"
        want = a_ref.float() @ w.float().t() + bias + res.float()
        err = ((out.float() - want).norm() / want.norm()).item()
        assert err < 6e-3, f"rank {r}: rel err {err}"
        s0 += seq[r]


def test_single_rank():
    run_world([300], [4], 512)


def test_three_ranks_uneven():
    run_world([200, 77, 150], [3, 2, 3], 384)


def test_batched_and_few_ctas():
    run_world([130, 260], [2, 2], 256, b=2, ctas=3)
