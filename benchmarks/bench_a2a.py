"""Detailed all-to-all benchmarks (the headline number lives in the repository's bench.py).

    torchrun --nproc-per-node N --master-addr 127.0.0.1 benchmarks/bench_a2a.py --mode stages
    modes: stages | zerocopy | padding | sweep | overlap | fp8 | link

Modes follow the reference's benchmark/bench_a2a.py:168-443 (stages, zerocopy, padding, sweep,
overlap, link). `link` is the ceiling every NVLink fraction in this repository is quoted against:
flat 64 MiB copies from rank r into rank (r+1) % N's memory through this library's own two data
paths (bulk copies, and 16-byte loads and stores), one flow and all N flows at once, with no
handshake and no relayout. `overlap` runs once per transport of the asynchronous call (the kernel, and
the copy engines) and also reports how much the GEMMs slow down while the exchange runs beside
them: an exchange on the SMs can hide itself by taking time from them, which is the question the
reference's `zerosm` mode (:446-637) asked of its copy engines.
BASE is the torch.distributed form (permute, all_to_all_single, permute). Every number is a CUDA
event time, L2 flushed between iterations, the maximum over ranks; rank 0 prints one JSON line
per measurement.
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

SHAPES = {  # name: (total tokens, heads, last dim) as in the reference's table (q, k, v packed: 3 * 128)
    "wan-720p": (75827, 40, 384),
    "wan-480p": (32987, 40, 384),
    "wan-720p-d128": (75600, 40, 128),
}


def timer(world, flush):
    def run(fn, iters=25, warmup=8):
        for _ in range(warmup):
            flush.zero_()
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        st = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
        en = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
        for i in range(iters):
            flush.zero_()
            st[i].record()
            fn()
            en[i].record()
        torch.cuda.synchronize()
        ms = sorted(a.elapsed_time(b) for a, b in zip(st, en))[iters // 2]
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    return run


def base_a2a(x, world):
    b, s, n, d = x.shape
    t = x.reshape(b, s, world, n // world, d).permute(2, 0, 1, 3, 4).contiguous()
    o = torch.empty_like(t)
    dist.all_to_all_single(o, t)
    return o.permute(1, 0, 2, 3, 4).reshape(b, world * s, n // world, d)


def emit(rank, **kw):
    if rank == 0:
        print(json.dumps(kw), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="stages", choices=["stages", "zerocopy", "padding", "sweep", "overlap", "fp8", "link"])
    ap.add_argument("--shape", default="wan-720p", choices=list(SHAPES))
    ap.add_argument("--iters", type=int, default=25)
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    g = fu.UlyssesGroup(device=torch.device("cuda", local), require_nvlink=False)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    run = timer(world, flush)
    total, heads, d = SHAPES[args.shape]
    s_local = (total + world - 1) // world
    x = torch.randn(1, s_local, heads, d, device="cuda", dtype=torch.bfloat16)

    if args.mode == "stages":
        _, st = g._timed(x)
        emit(rank, mode="stages", shape=args.shape, world=world, base_ms=run(lambda: base_a2a(x, world), args.iters),
             ours_ms=run(lambda: g.all_to_all_4d(x), args.iters), kernel_phases_ms=st)
    elif args.mode == "zerocopy":
        out = g.empty_output(x)
        emit(rank, mode="zerocopy", shape=args.shape, world=world, copying_ms=run(lambda: g.all_to_all_4d(x), args.iters),
             zero_copy_ms=run(lambda: g.all_to_all_4d(x, out=out), args.iters))
    elif args.mode == "padding":
        # even shards padded up vs. the true uneven shards (no padding moved at all)
        base = total // world
        seq = [base + (1 if p < total % world else 0) for p in range(world)]
        hs = [heads // world + (1 if p < heads % world else 0) for p in range(world)]
        xu = torch.randn(1, seq[rank], heads, d, device="cuda", dtype=torch.bfloat16)
        emit(rank, mode="padding", shape=args.shape, world=world, padded_ms=run(lambda: g.all_to_all_4d(x), args.iters),
             unpadded_ms=run(lambda: g.all_to_all_4d(xu, seq_splits=seq, head_splits=hs), args.iters))
    elif args.mode == "sweep":
        for s in (16, 64, 256, 1024, 4096, 9478, 16384):
            xs = torch.randn(1, s, heads, d, device="cuda", dtype=torch.bfloat16)
            ms = run(lambda: g.all_to_all_4d(xs), args.iters)
            crossed = xs.numel() * 2 * (world - 1) / world
            emit(rank, mode="sweep", s_local=s, world=world, ms=ms, gb_per_s_crossed=crossed / ms / 1e6)
    elif args.mode == "overlap":
        a = torch.randn(8192, 8192, device="cuda", dtype=torch.bfloat16)

        def gemms():
            for _ in range(3):
                a @ a

        # `x` is never written here, so the asynchronous call reads it in place (stage=False).
        # Two forms of the call: "copying" returns a fresh tensor (window + copy-out), "lend"
        # returns the window itself (nothing is copied out).
        def exchange(form):
            return g.all_to_all_4d_async(x, stage=False, lend=(form == "lend"))

        t_g = run(gemms, args.iters)
        want = g.all_to_all_4d(x).clone()
        # (name, transport, test flags): the last row hands the copies that stay on the device to
        # the driver's pitched copy as well (FU_A2A_CE_LOCAL_COPIES), for comparison
        rows = [("kernel", "kernel", 0), ("copy_engine", "copy_engine", 0), ("copy_engine+driver_local_copies", "copy_engine", 512)]
        for name, transport, test_flags in rows:
            g.set_async_transport(transport)
            g._handle.set_test_flags(test_flags)
            for form in ("copying", "lend"):
                assert torch.equal(exchange(form).wait(), want), (name, form)

                def alone():
                    exchange(form).wait()

                def serial():
                    gemms()
                    exchange(form).wait()

                def concurrent():
                    h = exchange(form)
                    gemms()
                    h.wait()

                t_a = run(alone, args.iters)
                t_s, t_c = run(serial, args.iters), run(concurrent, args.iters)
                # how long the GEMMs themselves take while the exchange runs beside them (events around
                # the GEMMs only, on the caller's stream): an exchange can hide itself by taking SMs from them
                pairs = []
                for _ in range(args.iters):
                    flush.zero_()
                    h = exchange(form)
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    gemms()
                    e1.record()
                    h.wait()
                    pairs.append((e0, e1))
                torch.cuda.synchronize()
                beside = sorted(p0.elapsed_time(p1) for p0, p1 in pairs)[len(pairs) // 2]
                tb = torch.tensor([beside], device="cuda", dtype=torch.float64)
                dist.all_reduce(tb, op=dist.ReduceOp.MAX)
                emit(rank, mode="overlap", transport=name, form=form, shape=args.shape, world=world, gemm_ms=t_g, a2a_ms=t_a,
                     serial_ms=t_s, concurrent_ms=t_c, hidden_pct=100.0 * (t_s - t_c) / t_a,
                     gemm_beside_exchange_ms=float(tb), gemm_slowdown_pct=100.0 * (float(tb) - t_g) / t_g)
        g._handle.set_test_flags(0)
    elif args.mode == "fp8":
        from fast_ulysses_b200.ops import fp8

        x128 = torch.randn(1, s_local, heads, 128, device="cuda", dtype=torch.bfloat16)
        x8 = torch.randint(-128, 127, (1, s_local, heads, 128), device="cuda", dtype=torch.int8)
        # the block-scaled time includes the quantise and dequantise kernels around the exchange
        emit(rank, mode="fp8", world=world, bf16_ms=run(lambda: g.all_to_all_4d(x128), args.iters),
             fp8_block_scaled_ms=run(lambda: fp8.all_to_all_4d_fp8(g, x128), args.iters),
             int8_payload_ms=run(lambda: g.all_to_all_4d(x8), args.iters))
    elif args.mode == "link":
        import ctypes as C

        from fast_ulysses_b200.ops import _ckernels as ck

        nbytes = 64 << 20
        buf = g._handle.symm_alloc(nbytes)  # collective: every rank's buffer, mapped on every rank
        ptrs = g._handle.symm_ptrs(buf)
        bases, ctrls = ptrs[:world], ptrs[world:]
        src = torch.full((nbytes,), 1, dtype=torch.uint8, device="cuda")
        peer = (rank + 1) % world

        def flat(flags):
            a = ck.FuA2AArgs()
            a.src = src.data_ptr()
            for p in range(world):
                a.peer_win[p], a.peer_ctrl[p] = bases[p], ctrls[p]
            a.rank, a.world, a.n_routes = rank, world, 1
            a.routes[0] = ck.FuRoute(peer, 0, 0, 0, nbytes, nbytes, nbytes, 1, 1, 0, 0)
            a.flags = ck.FU_A2A_NO_HANDSHAKE | flags
            a.win_bytes, a.src_bytes = nbytes, nbytes
            ck.check(ck.lib().fu_a2a4d(C.byref(a), ck.stream_ptr()))

        for name, flags in (("bulk", 0), ("ldst", ck.FU_A2A_LDST)):
            if world == 1:
                emit(rank, mode="link", path=name, note="world_size 1: no link to measure")
                continue
            one = run(lambda: flat(flags) if rank == 0 else None, args.iters)  # a single flow on the fabric
            every = run(lambda: flat(flags), args.iters)                      # one flow per rank
            emit(rank, mode="link", path=name, world=world, bytes=nbytes, one_flow_ms=one,
                 one_flow_gb_per_s=nbytes / one / 1e6, all_flows_ms=every, per_flow_gb_per_s=nbytes / every / 1e6,
                 aggregate_gb_per_s=world * nbytes / every / 1e6)
        del buf
    g.check()
    g.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
