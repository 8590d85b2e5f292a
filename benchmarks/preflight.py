"""The manual gate before a release: build, `doctor`, and the GPU test suites on a real machine.

    python benchmarks/preflight.py                 # every GPU nvidia-smi reports
    python benchmarks/preflight.py --gpus 0,1,2,3  # a subset

CI has no GPU runner: `.github/workflows/ci.yml` cross-compiles for sm_100a and runs the CPU and
gloo tests, and stops there. Everything that touches a device (the symmetric windows, the
handshakes, the fused kernels) is only exercised here, so a release cut without this run is
untested. The steps, each with its exit status in the summary block at the end:

  1. in-tree build of both libraries for sm_100a (`fast_ulysses_b200._build`)
  2. `python -m fast_ulysses_b200 doctor` (build facts, architecture of the visible GPUs, NVLink matrix)
  3. the single-GPU suite, `pytest tests -m gpu` without the multi-GPU file
  4. the multi-GPU suite, `pytest tests/test_multigpu.py`, under `benchmarks/exclusive.py`, which
     refuses a machine that other compute processes are using and says at the end whether the
     GPUs stayed ours: pass/fail and numbers from a contended box are both worthless

Read-only with respect to the machine: nothing here sets clocks, power limits or modes. The
counterpart in the reference is tools/preflight_gpu.sh:1-129, which additionally installs a wheel
into a clean virtualenv; this library builds in-tree for one toolchain and has no wheel matrix.
"""

from __future__ import annotations

import argparse
import os
import platform
import re
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def run(cmd: list[str], env: dict | None = None) -> tuple[int, str]:
    """Runs `cmd` from the repository root, echoing its output; returns (exit status, output)."""
    print("$", " ".join(cmd), flush=True)
    proc = subprocess.Popen(cmd, cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    lines = []
    for line in proc.stdout:
        sys.stdout.write(line)
        lines.append(line)
    return proc.wait(), "".join(lines)


def last_match(pattern: str, text: str) -> str:
    found = [ln.strip() for ln in text.splitlines() if re.search(pattern, ln)]
    return found[-1] if found else "unreported"


def smi(field: str) -> list[str]:
    try:
        out = subprocess.run(["nvidia-smi", f"--query-gpu={field}", "--format=csv,noheader"], capture_output=True,
                             text=True)
        return [ln.strip() for ln in out.stdout.splitlines() if ln.strip()]
    except OSError:
        return []


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", default=None, help="comma-separated indices (default: all)")
    ap.add_argument("--skip-single", action="store_true", help="skip the single-GPU suite")
    args = ap.parse_args()
    indices = smi("index")
    gpus = args.gpus or ",".join(indices)
    if not gpus:
        print("preflight needs a machine with GPUs (nvidia-smi reported none)")
        return 2
    py = sys.executable
    env = dict(os.environ, CUDA_VISIBLE_DEVICES=gpus)

    build_rc, _ = run([py, "-m", "fast_ulysses_b200._build", "-q"])
    doctor_rc, doctor_out = run([py, "-m", "fast_ulysses_b200", "doctor"], env)
    single_rc, single_out = (0, "skipped") if args.skip_single else run(
        [py, "-m", "pytest", "tests", "-m", "gpu", "-q", "--ignore=tests/test_multigpu.py"], env)
    multi_rc, multi_out = run([py, "benchmarks/exclusive.py", "--gpus", gpus, "--", py, "-m", "pytest",
                               "tests/test_multigpu.py", "-q"])

    import torch

    names, drivers = smi("name"), smi("driver_version")
    tally = r"passed|failed|error|skipped|no tests ran"
    status = lambda rc: "ok" if rc == 0 else f"FAILED (exit {rc})"  # noqa: E731
    print(f"""
--- paste into the release notes ---
Preflight (manual; the GPU suites have no CI runner)
  host        : {platform.node()}, {len(indices)} x {names[0] if names else '?'}, driver {drivers[0] if drivers else '?'}
  gpus used   : {gpus}
  python      : {platform.python_version()}
  torch       : {torch.__version__} (CUDA {torch.version.cuda})
  build       : {status(build_rc)}
  doctor      : {status(doctor_rc)}
  nvlink      : {last_match(r'NVLink|no pair to check|could not report', doctor_out)}
  single GPU  : {status(single_rc)} -- {last_match(tally, single_out)}
  multi GPU   : {status(multi_rc)} -- {last_match(tally, multi_out)}
  exclusivity : {last_match(r'^(EXCLUSIVE|CONTENDED)', multi_out)}
------------------------------------""")
    # exclusive.py exits 3 (refused) or 4 (contended) without the suite having proven anything, so a
    # non-zero status is never "the build is fine, the box was busy": run it again
    return 0 if build_rc == doctor_rc == single_rc == multi_rc == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
