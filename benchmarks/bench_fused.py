"""Each fused compute+collective kernel of the attention block on its own, over real NVLink.

    torchrun --nproc-per-node N --master-addr 127.0.0.1 benchmarks/bench_fused.py [--tokens 75600]

Wan2.1-14B shape (hidden 5120, 40 heads x 128, 75600 tokens split evenly over the N ranks). For every
kernel: CUDA-event time (median of `--iters` after a warm-up, L2 flushed between launches, maximum
over ranks) and the fraction of its roofline, defined as the slower of
  * its FLOPs at the measured cuBLAS bf16 rate of this pool (`bf16_tflops` of MEASURED_PEAKS.json,
    burst figure: the kernel is timed in isolation), and
  * the bytes that must cross NVLink at the measured peer-copy rate: `--link-gbs`, which should be
    the per-flow figure that `benchmarks/bench_a2a.py --mode link` printed on the same machine
    (default 636, what that mode measured for one flow through the bulk path at 4 and 8 GPUs of this pool), and
  * for the memory-bound gradient pull, its local HBM bytes at the measured copy rate (`hbm_gbs`).
Rank 0 prints one JSON line per kernel. Nothing here runs under a profiler.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

import fast_ulysses_b200 as fu
from fast_ulysses_b200.models.attention import HEAD_DIM, UlyssesSelfAttention
from fast_ulysses_b200.ops import attention as fa
from fast_ulysses_b200.ops import gemm, outproj, qkv


def peaks() -> tuple[float, float]:
    """(cuBLAS bf16 TFLOP/s, copy GB/s) as measured on this pool, or the pool's stated fallback."""
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        d = json.load(open(path))
        return float(d["bf16_tflops"]), float(d["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        return 1590.0, 6650.0


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=75600)
    ap.add_argument("--iters", type=int, default=15)
    ap.add_argument("--link-gbs", type=float, default=636.0)
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    g = fu.UlyssesGroup(device=torch.device("cuda", local), require_nvlink=False)
    hidden, heads = 5120, 40
    assert args.tokens % world == 0 and heads % world == 0
    torch.manual_seed(1)
    mod = UlyssesSelfAttention(g, hidden, heads, grid=(1, 1, args.tokens))
    m, n_local = mod.s_local, mod.n_local
    x = torch.randn(m, hidden, device="cuda").bfloat16()
    dy = torch.randn(m, hidden, device="cuda").bfloat16()
    y_save = torch.empty(m, 2 * heads * HEAD_DIM, dtype=torch.bfloat16, device="cuda")
    gather = torch.empty(m, heads * HEAD_DIM, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(m, hidden, dtype=torch.bfloat16, device="cuda")
    dyqkv = torch.empty(m, 3 * heads * HEAD_DIM, dtype=torch.bfloat16, device="cuda")
    dgq, dgk = torch.zeros(HEAD_DIM, device="cuda"), torch.zeros(HEAD_DIM, device="cuda")
    gq, gk = mod._f32("gamma_q", mod.gamma_q), mod._f32("gamma_k", mod.gamma_k)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    (tflops, hbm), link = peaks(), args.link_gbs
    remote = (world - 1) / world  # share of a rank's rows or heads that lives on other ranks

    def timed(fn):
        for _ in range(3):
            flush.zero_()
            fn()
        gemm.check_errors()
        g.check()
        torch.cuda.synchronize()
        dist.barrier()
        st = [torch.cuda.Event(enable_timing=True) for _ in range(args.iters)]
        en = [torch.cuda.Event(enable_timing=True) for _ in range(args.iters)]
        for i in range(args.iters):
            flush.zero_()
            st[i].record()
            fn()
            en[i].record()
        torch.cuda.synchronize()
        ms = sorted(a.elapsed_time(b) for a, b in zip(st, en))[args.iters // 2]
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def report(name, ms, flops, nvlink_bytes, hbm_bytes=0.0):
        t = {"compute": flops / (tflops * 1e9), "nvlink": nvlink_bytes / (link * 1e6), "hbm": hbm_bytes / (hbm * 1e6)}  # ms
        bound = max(t, key=t.get)
        if rank == 0:
            print(json.dumps({"kernel": name, "world": world, "ms": round(ms, 4), "compute_ms_at_peak": round(t["compute"], 4),
                              "nvlink_ms_at_link_rate": round(t["nvlink"], 4), "hbm_ms_at_copy_rate": round(t["hbm"], 4),
                              "roofline_fraction": round(t[bound] / ms, 3), "bound": bound}), flush=True)

    row_bytes = heads * HEAD_DIM * 2
    # fused QKV projection + RMSNorm + RoPE + scatter: 3 x (m, hidden) of results leave for the head owners
    ms = timed(lambda: mod._launch_scatter(x, mod.w_qkv, mod.qkv_win, 3, 2, mod.gamma_q, mod.gamma_k, y_save))
    report("qkv_rope_scatter", ms, 2.0 * m * 3 * heads * HEAD_DIM * hidden, 3 * m * row_bytes * remote)
    # attention on this rank's heads over the whole sequence (no collective; for the block's budget)
    ms = timed(lambda: fa.fmha_fwd(mod.q_view, mod.k_view, mod.v_view, out=mod.o_view))
    report("fmha_fwd", ms, 4.0 * args.tokens * args.tokens * HEAD_DIM * n_local, 0.0)
    _, lse = fa.fmha_fwd(mod.q_view, mod.k_view, mod.v_view, out=mod.o_view)
    # pull + output projection: the attention output of this rank's tokens comes from the head owners
    ready = mod._ready_flags(m)
    ms = timed(lambda: outproj.pull_outproj_raw(mod.w_o, out, gather, ready, s_local=m, seq_off=mod.seq_off,
                                                s_total=mod.s_total, head_splits=mod.head_splits, rank=mod.rank,
                                                peer_o=mod.o_buf.base, ctrl=mod.o_buf.ctrl, o_bytes=mod._region))
    report("pull_outproj", ms, 2.0 * m * hidden * heads * HEAD_DIM, m * row_bytes * remote)
    # backward: d(attention output) scattered from the dgrad GEMM's epilogue
    ms = timed(lambda: mod._launch_scatter(dy, mod.w_o, mod.do_win, 1, 0, None, None, None, w_kn=True))
    report("dout_scatter", ms, 2.0 * m * hidden * heads * HEAD_DIM, m * row_bytes * remote)
    ms = timed(lambda: fa.fmha_bwd(mod.q_view, mod.k_view, mod.v_view, mod.o_view, lse, mod.do_view,
                                   out=(mod.dq_view, mod.dk_view, mod.dv_view)))
    report("fmha_bwd", ms, 10.0 * args.tokens * args.tokens * HEAD_DIM * n_local, 0.0)
    # dq, dk, dv pulled home with RoPE and RMSNorm undone on the way (memory-bound: no FLOPs to speak of)
    R = mod._region
    ms = timed(lambda: qkv.pull_qkv_grads_raw(dyqkv, y_save, mod.rope, gq, gk, dgq, dgk, heads=heads, s_local=m,
                                              seq_off=mod.seq_off, s_total=mod.s_total, head_splits=mod.head_splits,
                                              rank=mod.rank, peer_dq=mod.dqkv_buf.base,
                                              peer_dk=[p + R for p in mod.dqkv_buf.base],
                                              peer_dv=[p + 2 * R for p in mod.dqkv_buf.base], ctrl=mod.dqkv_buf.ctrl,
                                              src_bytes=R))
    # local HBM sees: the share of dq/dk/dv this GPU serves (to itself and to peers), the saved pre-norm
    # rows of q and k, and the three projections' gradients written
    report("pull_qkv_grads", ms, 0.0, 3 * m * row_bytes * remote, hbm_bytes=8.0 * m * row_bytes)
    g.check()
    g.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
