"""Block-scaled fp8 payloads: the CPU statement of the format everywhere, the CUDA kernels against
it on a GPU, and the exchange on the CPU/gloo backend with uneven shards."""

import pytest
import torch

from fast_ulysses_b200.ops import fp8


def test_cpu_round_trip_error_is_fp8_sized():
    torch.manual_seed(0)
    x = (torch.randn(2, 37, 5, 128) * torch.rand(2, 37, 5, 1) * 10).bfloat16()
    x[0, 0, 0] = 0  # an all-zero block keeps scale 1
    p = fp8.quantize(x)
    assert p.shape == (2, 37, 5, 144) and p.dtype == torch.uint8
    y = fp8.dequantize(p)
    amax = x.float().abs().amax(-1, keepdim=True).clamp_min(1e-30)
    assert ((y.float() - x.float()).abs() / amax).max() < 0.07  # e4m3: 3 mantissa bits
    assert torch.all(y[0, 0, 0] == 0)


@pytest.mark.gpu
def test_cuda_kernels_match_the_cpu_statement():
    torch.manual_seed(1)
    x = (torch.randn(3, 50, 4, 128, device="cuda") * 5).bfloat16()
    p_gpu = fp8.quantize(x)
    p_cpu = fp8.quantize(x.cpu())
    # scales are identical; payload bytes may differ by one rounding step where x/scale sits on a tie
    assert torch.equal(p_gpu[..., 128:132].cpu(), p_cpu[..., 128:132])
    diff = (fp8.dequantize(p_gpu).float().cpu() - fp8.dequantize(p_cpu).float()).abs()
    assert diff.max() <= 0.13 * x.float().abs().max().item()
    assert (diff > 0).float().mean() < 0.02
    y = fp8.dequantize(p_gpu)
    amax = x.float().abs().amax(-1, keepdim=True)
    assert ((y.float() - x.float()).abs() / amax).max() < 0.07
    assert torch.equal(fp8.dequantize(p_cpu.cuda()), fp8.dequantize(p_cpu).cuda())


def test_exchange_with_scales_over_gloo():
    from _dist import run_ranks

    run_ranks(3, "_gloo_workers", "fp8_exchange")


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [0, 1])
def test_fused_exchange_kernel_matches_quantise_permute_dequantise(mode):
    """fu_a2a4d_fp8 on one device with three emulated ranks (uneven shards, handshakes off) against
    the statement of what it computes: quantise every row, move it where the all-to-all puts it,
    dequantise. Launched twice per rank: the first round fills every window, the second expands
    complete windows."""
    import ctypes as C

    import fast_ulysses_b200  # noqa: F401  (registers the torch ops)
    from fast_ulysses_b200.ops import _ckernels as ck

    torch.manual_seed(5 + mode)
    b, seq, heads = 2, [17, 40, 9], [14, 13, 13]
    ws, S, N = len(seq), sum(seq), sum(heads)
    glob = (torch.randn(b, S, N, 128, device="cuda") * torch.rand(b, S, N, 1, device="cuda") * 6).bfloat16()
    s0 = [sum(seq[:p]) for p in range(ws)]
    h0 = [sum(heads[:p]) for p in range(ws)]
    by_seq = [glob[:, s0[p]:s0[p] + seq[p]].contiguous() for p in range(ws)]
    by_head = [glob[:, :, h0[p]:h0[p] + heads[p]].contiguous() for p in range(ws)]
    inputs, expected = (by_seq, by_head) if mode == 0 else (by_head, by_seq)
    plans = [torch.ops.fast_ulysses_b200.a2a_plan_debug(b, 128, r, ws, seq, heads, mode, 2) for r in range(ws)]
    win_bytes = plans[0][1] // 128 * 144
    wins = [torch.zeros(win_bytes + ck.FU_CTRL_BYTES, dtype=torch.uint8, device="cuda") for _ in range(ws)]
    outs = [torch.zeros(tuple(plans[r][0]), dtype=torch.bfloat16, device="cuda") for r in range(ws)]
    for _ in range(2):
        for r in range(ws):
            a = ck.FuA2AFp8Args()
            a.src, a.out = inputs[r].data_ptr(), outs[r].data_ptr()
            for p in range(ws):
                a.peer_win[p], a.peer_ctrl[p] = wins[p].data_ptr(), wins[p].data_ptr() + win_bytes
            a.win_bytes, a.src_bytes, a.out_rows = win_bytes, inputs[r].numel() * 2, outs[r].numel() // 128
            a.rank, a.world, a.flags = r, ws, ck.FU_A2A_NO_HANDSHAKE
            rows = plans[r][2].tolist()
            a.n_routes = len(rows)
            for i, row in enumerate(rows):
                a.routes[i] = ck.route_from_row(row)
            ck.check(ck.lib().fu_a2a4d_fp8(C.byref(a), ck.stream_ptr()))
    torch.cuda.synchronize()
    for r in range(ws):
        want = fp8.dequantize(fp8.quantize(expected[r]))
        assert outs[r].shape == want.shape and torch.equal(outs[r], want), f"rank {r}"
