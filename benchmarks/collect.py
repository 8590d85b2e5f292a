"""Runs every benchmark mode and writes one log with a fingerprint header (host, commit, driver,
torch, clocks before/after, topology, doctor), like the reference's benchmark/collect.sh:35-139.
Read-only with respect to the GPUs.

    python benchmarks/collect.py --gpus 8 --out results.log [--skip-tests]
"""

from __future__ import annotations

import argparse
import datetime
import os
import platform
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MODES = ["link", "stages", "zerocopy", "padding", "sweep", "overlap", "fp8"]


def sh(cmd: list[str]) -> str:
    try:
        return subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=1800).stdout.strip()
    except Exception as e:  # a missing tool must not stop the collection
        return f"<{type(e).__name__}: {e}>"


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--out", default="bench_results.log")
    ap.add_argument("--skip-tests", action="store_true")
    args = ap.parse_args()
    clocks = ["nvidia-smi", "--query-gpu=index,clocks.sm,clocks.max.sm,power.draw", "--format=csv"]
    with open(args.out, "w") as f:
        def w(title, body):
            f.write(f"==== {title}\n{body}\n")
            f.flush()

        w("when / host", f"{datetime.datetime.now(datetime.timezone.utc).isoformat()}  {platform.node()}")
        w("commit", sh(["git", "rev-parse", "HEAD"]))
        w("driver / gpus", sh(["nvidia-smi", "--query-gpu=index,name,driver_version", "--format=csv"]))
        w("torch", sh([sys.executable, "-c", "import torch; print(torch.__version__, torch.version.cuda)"]))
        w("clocks before", sh(clocks))
        w("topology", sh(["nvidia-smi", "topo", "-m"]))
        w("doctor", sh([sys.executable, "-m", "fast_ulysses_b200", "doctor"]))
        failed = []
        if not args.skip_tests:
            out = sh([sys.executable, "-m", "pytest", "tests", "-q", "-m", "gpu"])
            w("correctness gate (pytest -m gpu)", out[-2000:])
            if " failed" in out:
                failed.append("tests")
        run = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1"]
        for mode in MODES:
            out = sh(run + ["benchmarks/bench_a2a.py", "--mode", mode])
            w(f"bench_a2a --mode {mode} ({args.gpus} GPUs)", "\n".join(l for l in out.splitlines() if l.startswith("{")))
            if "{" not in out:
                failed.append(mode)
        out = sh(run + ["benchmarks/bench_fused.py"])
        w(f"bench_fused ({args.gpus} GPUs)", "\n".join(l for l in out.splitlines() if l.startswith("{")))
        w("headline (bench.py)", sh(run + ["bench.py", "--gpus", str(args.gpus)])[-3000:])
        w("clocks after", sh(clocks))
        w("failed modes", ", ".join(failed) or "none")
    print(f"wrote {args.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
