"""Was the GPU ours while the benchmark ran?  Read-only: queries nvidia-smi, changes nothing.

    python benchmarks/exclusive.py --gpus 0,1 -- <command ...>

Refuses to start (exit 3) while other compute processes are on the requested GPUs, samples the
foreign process count and the minimum SM clock while the command runs, and prints
``EXCLUSIVE`` or ``CONTENDED`` (exit 4) at the end. Counterpart of the reference's
tools/exclusive.sh:96-113; it never sets clocks, power limits or modes."""

from __future__ import annotations

import argparse
import os
import subprocess
import sys
import threading
import time


def smi(query: str, gpus: str) -> list[list[str]]:
    out = subprocess.run(["nvidia-smi", f"--query-{query}", "--format=csv,noheader,nounits", "-i", gpus],
                         capture_output=True, text=True)
    return [[c.strip() for c in line.split(",")] for line in out.stdout.splitlines() if line.strip()]


def foreign_pids(gpus: str, own: set[int]) -> set[int]:
    rows = smi("compute-apps=pid,gpu_uuid", gpus)
    return {int(r[0]) for r in rows if r and r[0].isdigit() and int(r[0]) not in own}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", default="0")
    ap.add_argument("--sample-secs", type=float, default=0.5)
    ap.add_argument("cmd", nargs=argparse.REMAINDER)
    args = ap.parse_args()
    cmd = args.cmd[1:] if args.cmd[:1] == ["--"] else args.cmd
    if not cmd:
        ap.error("no command given")
    if foreign_pids(args.gpus, set()):
        print("CONTENDED before start: other compute processes are on the requested GPUs")
        return 3
    env = dict(os.environ, CUDA_VISIBLE_DEVICES=args.gpus)
    proc = subprocess.Popen(cmd, env=env)
    seen_foreign, min_clock = 0, None
    stop = threading.Event()

    def sample():
        nonlocal seen_foreign, min_clock
        while not stop.is_set():
            try:
                import psutil

                own = {proc.pid} | {c.pid for c in psutil.Process(proc.pid).children(recursive=True)}
            except Exception:
                own = {proc.pid}
            seen_foreign = max(seen_foreign, len(foreign_pids(args.gpus, own)))
            for row in smi("gpu=clocks.sm", args.gpus):
                if row and row[0].isdigit():
                    min_clock = int(row[0]) if min_clock is None else min(min_clock, int(row[0]))
            time.sleep(args.sample_secs)

    t = threading.Thread(target=sample, daemon=True)
    t.start()
    rc = proc.wait()
    stop.set()
    t.join(timeout=2)
    verdict = "EXCLUSIVE" if seen_foreign == 0 else "CONTENDED"
    print(f"{verdict}: foreign compute processes seen {seen_foreign}, minimum SM clock {min_clock} MHz, exit {rc}")
    return rc if rc else (0 if seen_foreign == 0 else 4)


if __name__ == "__main__":
    sys.exit(main())
