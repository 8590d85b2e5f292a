"""Headline benchmark: ms per Wan-720p bf16 ``all_to_all_4d`` (and, where built, the
sequence-parallel attention block), device-timed, max over ranks.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N ...            # the unmodified reference build

For N > 1 launch with ``python -m torch.distributed.run --nnodes=1 --nproc-per-node N ...``.
Rank 0 prints exactly one JSON line.

Config (the one the baseline names): 81 frames -> 21x45x80 = 75600 tokens in total, split evenly
over the N ranks, 40 heads, d = 128, bf16, b = 1, mode 0 (scatter heads, gather sequence) through
the public copying call. Total work is fixed as N grows (strong scaling). Timing: CUDA events
around every step, L2 flushed between steps by writing a 256 MiB buffer, a barrier and a device
synchronise on both sides of the timed region. The reported value is the median over the timed
steps of each rank, maximum over ranks (the reference's own method: benchmark/bench_a2a.py:101-123
takes medians after a warm-up); mean, minimum, maximum, the slowest step and the rank that owned it
are printed beside it so that an outlier shows. The warm-up runs the requested number of steps and
then keeps going until at least 30 ms of device time of the step itself have passed, the same rule
in both arms, and the clock sampler has delivered its first row before any of that starts.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
TOTAL_TOKENS, HEADS, HEAD_DIM = 75600, 40, 128
PUBLISHED_MS = {8: 0.550, 4: 0.808}  # packed d=384 shape, reference README.md:37, docs/benchmark.md:202


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.first = index, [], None, 0

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None
            return
        # nvidia-smi attaches to every GPU of the box while it starts; let that finish before
        # anything is timed, so that its start-up never runs beside a timed step
        t_end = time.time() + 20.0
        while not self.rows and time.time() < t_end and self.proc.poll() is None:
            time.sleep(0.05)

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def mark(self):
        """Rows from here on belong to the timed region."""
        self.first = len(self.rows)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()  # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows[self.first:] or self.rows[-1:]:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def setup_dist(n: int):
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    if world > 1 or n > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    return rank, local, world


def max_over_ranks(v: float, world: int) -> float:
    if world == 1:
        return v
    t = torch.tensor([v], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sync_all(world: int):
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


MIN_WARM_MS = 30.0  # device time of the step itself that the warm-up must cover, in both arms


def gather_rows(vals, world: int):
    """Every rank's list of floats, as a list of lists indexed by rank (the same on every rank)."""
    if world == 1:
        return [list(vals)]
    mine = torch.tensor(vals, device="cuda", dtype=torch.float64)
    rows = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(rows, mine)
    return [r.tolist() for r in rows]


def run_timed(step, n: int, flush: torch.Tensor):
    """Per-step device times (ms) of n steps, each preceded by an L2 flush outside its event pair."""
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
    for i in range(n):
        flush.zero_()
        starts[i].record()
        step()
        ends[i].record()
    torch.cuda.synchronize()
    return [s.elapsed_time(e) for s, e in zip(starts, ends)]


def time_steps_stats(step, steps: int, warmup: int, world: int, flush: torch.Tensor) -> dict:
    """Device time per step. `ms` is the median over the timed steps of a rank, maximum over ranks."""
    warm = run_timed(step, warmup, flush)
    # keep warming until MIN_WARM_MS of the step's own device time have passed; every rank derives the
    # same number of extra steps from the same gathered figures, so collectives stay matched
    per_step = max(statistics.median(r) for r in gather_rows(warm, world))
    done = per_step * warmup
    extra_warm = 0 if done >= MIN_WARM_MS else min(2000, int((MIN_WARM_MS - done) / max(per_step, 1e-3)) + 1)
    for _ in range(extra_warm):
        flush.zero_()
        step()
    sync_all(world)
    rows = gather_rows(run_timed(step, steps, flush), world)
    sync_all(world)
    medians = [statistics.median(r) for r in rows]
    worst_rank = max(range(world), key=lambda r: max(rows[r]))
    worst_step = max(range(steps), key=lambda i: rows[worst_rank][i])
    return {"ms": max(medians), "mean_ms": max(sum(r) / len(r) for r in rows), "min_ms": min(min(r) for r in rows),
            "max_ms": rows[worst_rank][worst_step], "slowest_step": worst_step, "slowest_rank": worst_rank,
            "median_by_rank": [round(m, 5) for m in medians], "warmup_steps_run": warmup + extra_warm}


def time_steps(step, steps: int, warmup: int, world: int, flush: torch.Tensor) -> float:
    """ms per step: median over steps, maximum over ranks (see time_steps_stats)."""
    return time_steps_stats(step, steps, warmup, world, flush)["ms"]


def make_group(impl: str, local: int, world: int):
    if impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import fast_ulysses  # the unmodified reference build

        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29512")
            dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", local))
        return fast_ulysses.UlyssesGroup(device=torch.device("cuda", local), require_nvlink=False)
    import fast_ulysses_b200 as fu

    return fu.UlyssesGroup(device=torch.device("cuda", local), require_nvlink=False)


def reference_block(group, world, rank, time_steps, flush, steps=5, warmup=3) -> dict:
    """The composed baseline for the attention block: the reference's all_to_all_4d around
    nn.Linear (cuBLAS), separate RMSNorm / RoPE elementwise kernels and torch SDPA, as in the
    reference's examples/dit_attention.py. None of this repository's kernels are on this path."""
    import math

    grid, hidden, heads, d = (21, 45, 80), 5120, 40, 128
    total = grid[0] * grid[1] * grid[2]
    s_local, n_local = total // world, heads // world
    dev = group.device
    torch.manual_seed(1234)
    qkv = torch.nn.Linear(hidden, 3 * hidden, bias=False, device=dev, dtype=torch.bfloat16)
    proj = torch.nn.Linear(hidden, hidden, bias=True, device=dev, dtype=torch.bfloat16)
    gq = torch.nn.Parameter(torch.ones(d, device=dev, dtype=torch.bfloat16))
    gk = torch.nn.Parameter(torch.ones(d, device=dev, dtype=torch.bfloat16))
    idx = torch.arange(rank * s_local, (rank + 1) * s_local, device=dev)
    pos = (idx // (grid[1] * grid[2]), (idx // grid[2]) % grid[1], idx % grid[2])
    ang = torch.cat([p_.double()[:, None] / (10000.0 ** (torch.arange(0, n, 2, device=dev).double() / n))[None, :]
                     for p_, n in zip(pos, (44, 42, 42))], dim=1)
    cos, sin = ang.cos().to(torch.bfloat16)[None, :, None, :], ang.sin().to(torch.bfloat16)[None, :, None, :]

    def norm_rope(t, g):
        t = t * torch.rsqrt(t.float().pow(2).mean(-1, keepdim=True) + 1e-6).to(t.dtype) * g
        t2 = t.reshape(*t.shape[:-1], d // 2, 2)
        x0, x1 = t2[..., 0], t2[..., 1]
        return torch.stack((x0 * cos - x1 * sin, x0 * sin + x1 * cos), dim=-1).reshape(t.shape)

    def block(x):
        q, k, v = (t.reshape(1, s_local, heads, d) for t in qkv(x).chunk(3, dim=-1))
        q, k = norm_rope(q, gq), norm_rope(k, gk)
        q, k, v = (group.all_to_all_4d(t.contiguous(), mode=0) for t in (q, k, v))
        o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        o = group.all_to_all_4d(o.transpose(1, 2).contiguous(), mode=1)
        return proj(o.reshape(1, s_local, hidden))

    x = torch.randn(1, s_local, hidden, device=dev, dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn(1, s_local, hidden, device=dev, dtype=torch.bfloat16)
    params = list(qkv.parameters()) + list(proj.parameters()) + [gq, gk]

    def fwd():
        with torch.no_grad():
            block(x)

    def step():
        x.grad = None
        for p_ in params:
            p_.grad = None
        block(x).backward(dy)

    return {"fwd_ms": time_steps(fwd, steps, warmup, world, flush),
            "fwd_bwd_ms": time_steps(step, steps, warmup, world, flush),
            "config": {"composition": "reference all_to_all_4d + nn.Linear + torch norm/rope + torch SDPA"}}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary measurements")
    args = ap.parse_args()
    warmup = max(3, args.warmup)

    if args.impl == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "fast_ulysses")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref holds no installed reference build"}))
        return 0

    rank, local, world = setup_dist(args.gpus)
    try:
        group = make_group(args.impl, local, world)
    except Exception as e:  # the reference arm must report, not crash
        if args.impl == "reference":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}))
            return 0
        raise

    dev = torch.device("cuda", local)
    assert TOTAL_TOKENS % world == 0 and HEADS % world == 0, "bench.py runs even splits (N in 1, 2, 4, 8)"
    s_local = TOTAL_TOKENS // world
    torch.manual_seed(1234 + rank)
    x = torch.randn(1, s_local, HEADS, HEAD_DIM, device=dev, dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step():
        return group.all_to_all_4d(x, mode=0)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # returns once the first row has arrived
    sync_all(world)
    sampler.mark()
    head = time_steps_stats(step, args.steps, warmup, world, flush)
    ms = head["ms"]
    clocks = sampler.stop() if rank == 0 else {}

    # end to end: the step's input arrives from pinned host memory, its result is read back
    x_host = x.cpu().pin_memory()
    probe_host = torch.empty(1024, dtype=torch.bfloat16).pin_memory()
    x_dev = torch.empty_like(x)

    def e2e_step():
        x_dev.copy_(x_host, non_blocking=True)
        y = group.all_to_all_4d(x_dev, mode=0)
        probe_host.copy_(y.view(-1)[:1024], non_blocking=True)

    e2e = time_steps_stats(e2e_step, max(5, args.steps // 2), warmup, world, flush)
    e2e_ms = e2e["ms"]

    extra = {"headline_steps": head, "e2e_steps": e2e}
    if clocks.get("sm_mhz"):
        extra["headline_ms_x_sm_mhz"] = ms * clocks["sm_mhz"]
    if not args.no_extras:
        y = step()
        m1 = time_steps_stats(lambda: group.all_to_all_4d(y, mode=1), args.steps, warmup, world, flush)
        out = group.empty_output(x, mode=0)
        zc = time_steps_stats(lambda: group.all_to_all_4d(x, mode=0, out=out), args.steps, warmup, world, flush)
        extra["mode1_ms"], extra["mode1_steps"] = m1["ms"], m1
        extra["mode0_zero_copy_ms"], extra["mode0_zero_copy_steps"] = zc["ms"], zc
        del out, y
        if world in PUBLISHED_MS:
            # the shape the reference publishes: q, k, v packed (d = 384) with a 227-token text tail
            s_pack = (75827 + world - 1) // world
            xp = torch.randn(1, s_pack, HEADS, 3 * HEAD_DIM, device=dev, dtype=torch.bfloat16)
            t = time_steps(lambda: group.all_to_all_4d(xp, mode=0), args.steps, warmup, world, flush)
            extra["packed_d384"] = {"shape": [1, s_pack, HEADS, 3 * HEAD_DIM], "ms": t,
                                    "published_reference_ms": PUBLISHED_MS[world],
                                    "vs_published": t / PUBLISHED_MS[world]}
            del xp
        if args.impl == "ours":
            from fast_ulysses_b200.models.bench_block import bench_attention_block

            extra["sp_attention_block"] = bench_attention_block(group, world, rank, time_steps, flush)
        else:
            try:
                extra["sp_attention_block"] = reference_block(group, world, rank, time_steps, flush)
            except Exception as e:  # the composed baseline must not take the headline number down with it
                extra["sp_attention_block"] = {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
    if hasattr(group, "check"):
        group.check()

    if rank == 0:
        line = {
            "metric": "ms per Wan-720p bf16 all_to_all_4d (mode 0, copying call), max over ranks",
            "value": ms, "unit": "ms", "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms,
            "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (randn, seeded per rank)",
            "config": {"model": "Wan2.1-14B 720p attention exchange", "global_batch": 1, "seq_len": TOTAL_TOKENS,
                       "heads": HEADS, "head_dim": HEAD_DIM, "per_rank_shape": [1, s_local, HEADS, HEAD_DIM],
                       "parallelism": f"sp{world}", "l2": "flushed between steps (256 MiB write)",
                       "bytes_per_rank": x.numel() * 2, "statistic": "median over steps, max over ranks"},
            "copying_call": ("result returned in a pooled symmetric buffer written by the peers (library default; "
                             "group.set_output_pool(False) gives window + copy-out)")
            if args.impl == "ours" else "the reference's copying call",
            "clocks": clocks,
            "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": x.numel() * 2, "d2h_bytes_per_step": 2048},
            # one fused a2a4d kernel per timed step of the headline metric; the attention block in
            # `extra` launches 3 fused kernels forward and 9 kernels of this library backward
            "gpu_launches": args.steps if args.impl == "ours" else None,
            "extra": extra,
        }
        if args.impl == "reference":
            line["impl"] = "reference"
            line.pop("gpu_launches")
        if "packed_d384" in extra:
            line["vs_baseline"] = extra["packed_d384"]["vs_published"]
            line["vs_baseline_note"] = ("the published number is for the packed d=384 shape; vs_baseline compares "
                                        "extra.packed_d384.ms with it, not the d=128 value")
        print(json.dumps(line))
    group.destroy()
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
