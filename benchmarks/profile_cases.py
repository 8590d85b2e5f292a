"""Small single-GPU workloads, one per hot kernel, sized for a profiler capture: inputs larger than
L2 so that DRAM counters mean something, a few hundred MB on the device, one to three launches of
the kernel of interest after a short warm-up.

    python benchmarks/profile_cases.py a2a|gemm|gemm_pair|qkv|outproj|fmha_fwd|fmha_bwd|fmha_bwd_det

Each case prints the CUDA-event time of its last launch, so the same command is also a quick
timing check when run without a profiler.
"""

from __future__ import annotations

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _time(fn, warm=2, reps=2):
    from fast_ulysses_b200.ops import gemm as _gemm

    for i in range(warm):
        fn()
        if i == 0:
            _gemm.check_errors()  # a kernel that gave up on a wait takes seconds per launch: stop before looping
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ms = 0.0
    for _ in range(reps):
        t0.record()
        fn()
        t1.record()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1)
    return ms


def case_a2a():
    import fast_ulysses_b200 as fu

    g = fu.UlyssesGroup(device="cuda")
    x = torch.randn(1, 25000, 40, 128, device="cuda", dtype=torch.bfloat16)  # 256 MB
    ms = _time(lambda: g.all_to_all_4d(x))
    print(f"a2a4d single rank, 256 MB in -> 256 MB out: {ms:.4f} ms, {2 * x.numel() * 2 / ms / 1e6:.0f} GB/s r+w")


def case_gemm():
    from fast_ulysses_b200.ops import gemm

    a = torch.randn(8192, 8192, device="cuda").bfloat16()
    b = torch.randn(8192, 8192, device="cuda").bfloat16()
    ms = _time(lambda: gemm.gemm_bf16(a, b))
    print(f"gemm 8192^3: {ms:.4f} ms, {2 * 8192 ** 3 / ms / 1e9:.0f} TFLOP/s")


def case_gemm_pair():
    """The single-CTA kernel, the CTA-pair kernel and cuBLAS on 8192 cubed: median of 15 launches,
    256 MiB L2 flush before each."""
    from fast_ulysses_b200.ops import gemm

    a = torch.randn(8192, 8192, device="cuda").bfloat16()
    b = torch.randn(8192, 8192, device="cuda").bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for name, fn in (("single CTA", lambda: gemm.gemm_bf16(a, b, pair=False)),
                     ("CTA pairs", lambda: gemm.gemm_bf16(a, b, pair=True)), ("cuBLAS", lambda: a @ b.t())):
        for _ in range(5):
            fn()
        gemm.check_errors()
        times = []
        for _ in range(15):
            flush.zero_()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            fn()
            t1.record()
            torch.cuda.synchronize()
            times.append(t0.elapsed_time(t1))
        ms = sorted(times)[len(times) // 2]
        print(f"gemm 8192^3, {name}: {ms:.4f} ms, {2 * 8192 ** 3 / ms / 1e9:.0f} TFLOP/s")


def _fake_world(seq, head_splits, hidden):
    """Buffers for a single-device emulation of rank 0 of a world (handshakes off)."""
    from fast_ulysses_b200.ops import _ckernels as ck

    S, world = sum(seq), len(seq)
    region = S * max(head_splits) * 128 * 2
    wins = [torch.zeros(3 * region + ck.FU_CTRL_BYTES, dtype=torch.uint8, device="cuda") for _ in range(world)]
    return S, region, wins


def case_qkv():
    from fast_ulysses_b200.ops import _ckernels as ck
    from fast_ulysses_b200.ops import qkv
    from fast_ulysses_b200.ops.rope import rope_table

    # rank 0 of 8 at the Wan2.1-14B shape: M = 9450 rows, K = 5120, N = 3 * 40 * 128
    seq, hs, hidden, heads = [9450] * 8, [5] * 8, 5120, 40
    S, region, wins = _fake_world(seq, hs, hidden)
    x = torch.randn(9450, hidden, device="cuda").bfloat16()
    w = (torch.randn(3 * heads * 128, hidden, device="cuda") * 0.02).bfloat16()
    rope = rope_table(torch.arange(9450, device="cuda"))
    g = torch.ones(128, device="cuda")

    def run():
        qkv.qkv_rope_scatter_raw(x, w, rope, g, g, heads=heads, s_local=9450, seq_off=0, s_total=S, head_splits=hs,
                                 rank=0, win_q=[t.data_ptr() for t in wins],
                                 win_k=[t.data_ptr() + region for t in wins],
                                 win_v=[t.data_ptr() + 2 * region for t in wins],
                                 ctrl=[t.data_ptr() + 3 * region for t in wins], win_bytes=region,
                                 flags=ck.FU_A2A_NO_HANDSHAKE)

    ms = _time(run)
    print(f"fused qkv+rmsnorm+rope+scatter 9450x15360x5120: {ms:.4f} ms, {2 * 9450 * 15360 * 5120 / ms / 1e9:.0f} TFLOP/s")


def case_outproj():
    from fast_ulysses_b200.ops import _ckernels as ck
    from fast_ulysses_b200.ops import outproj

    hs, m, hidden = [5] * 8, 9450, 5120
    S = 8 * m
    o_bufs = [torch.randn(1, S, 5, 128, device="cuda").bfloat16() for _ in range(8)]
    ctrls = [torch.zeros(ck.FU_CTRL_BYTES, dtype=torch.uint8, device="cuda") for _ in range(8)]
    w = (torch.randn(hidden, 40 * 128, device="cuda") * 0.02).bfloat16()
    out = torch.empty(m, hidden, device="cuda", dtype=torch.bfloat16)
    gather = torch.empty(m, 40 * 128, device="cuda", dtype=torch.bfloat16)
    ready = torch.zeros(((m + 127) // 128) * 8, dtype=torch.int32, device="cuda")

    def run():
        outproj.pull_outproj_raw(w, out, gather, ready, s_local=m, seq_off=0, s_total=S, head_splits=hs, rank=0,
                                 peer_o=[t.data_ptr() for t in o_bufs], ctrl=[t.data_ptr() for t in ctrls],
                                 o_bytes=o_bufs[0].numel() * 2, flags=ck.FU_A2A_NO_HANDSHAKE)

    ms = _time(run)
    print(f"pull + out-proj 9450x5120x5120: {ms:.4f} ms, {2 * 9450 * 5120 * 5120 / ms / 1e9:.0f} TFLOP/s")


def _qkv_attn(S=16384, H=5):
    return tuple(torch.randn(1, S, H, 128, device="cuda").bfloat16() for _ in range(3))


def case_fmha_fwd():
    from fast_ulysses_b200.ops import attention

    q, k, v = _qkv_attn()
    ms = _time(lambda: attention.fmha_fwd(q, k, v))
    print(f"fmha fwd S=16384 H=5: {ms:.4f} ms, {4 * 16384 ** 2 * 128 * 5 / ms / 1e9:.0f} TFLOP/s")


def case_fmha_bwd():
    from fast_ulysses_b200.ops import attention

    q, k, v = _qkv_attn()
    o, lse = attention.fmha_fwd(q, k, v)
    d_o = torch.randn_like(o)
    ms = _time(lambda: attention.fmha_bwd(q, k, v, o, lse, d_o))
    print(f"fmha bwd S=16384 H=5: {ms:.4f} ms, {10 * 16384 ** 2 * 128 * 5 / ms / 1e9:.0f} TFLOP/s")


def case_fmha_bwd_det():
    from fast_ulysses_b200.ops import attention

    q, k, v = _qkv_attn()
    o, lse = attention.fmha_fwd(q, k, v)
    d_o = torch.randn_like(o)
    ms = _time(lambda: attention.fmha_bwd(q, k, v, o, lse, d_o, deterministic=True))
    print(f"fmha bwd (two passes, no atomics) S=16384 H=5: {ms:.4f} ms, {10 * 16384 ** 2 * 128 * 5 / ms / 1e9:.0f} TFLOP/s")


CASES = {"a2a": case_a2a, "gemm": case_gemm, "gemm_pair": case_gemm_pair, "qkv": case_qkv, "outproj": case_outproj, "fmha_fwd": case_fmha_fwd,
         "fmha_bwd": case_fmha_bwd, "fmha_bwd_det": case_fmha_bwd_det}

if __name__ == "__main__":
    name = sys.argv[1] if len(sys.argv) > 1 else ""
    if name not in CASES:
        sys.exit(f"usage: python benchmarks/profile_cases.py {'|'.join(CASES)}")
    CASES[name]()
    from fast_ulysses_b200.ops import gemm as _g

    _g.check_errors()
