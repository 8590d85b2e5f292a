"""``python -m fast_ulysses_b200 doctor``: what was built, what is installed, which GPUs are
visible, whether their architecture is the one this build targets, and the NVLink matrix.

Parity: python/fast_ulysses/cli.py:38-103 of the reference (`doctor`). Its `wheel-url` command
picks a wheel from a published matrix; this library is built in-tree for one architecture and has
no wheel matrix, so that command does not exist here.
"""

from __future__ import annotations

import argparse
import sys


def doctor(out=sys.stdout) -> int:
    """Prints the report; returns 0 when everything needed is present, 1 otherwise."""
    import torch

    try:
        import fast_ulysses_b200 as fu
    except ImportError as e:
        print(f"import failed:\n{e}", file=out)
        return 1
    from .diagnose import build_facts, live_facts

    info = fu._C.build_info()
    print(f"fast_ulysses_b200 {fu.__version__}", file=out)
    print(f"  extension : {fu._C.__file__}", file=out)
    print(f"  kernels   : {info['kernels']}", file=out)
    print(f"  built for : sm_{info['cuda_arch_list']}", file=out)
    built, live = build_facts(), live_facts()
    for key in ("torch", "cuda", "python"):
        mark = "" if built.get(key) in (None, live[key]) else f"   (built against {built[key]})"
        print(f"  {key:<9} : {live[key]}{mark}", file=out)
    rc = 0
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    print(f"devices ({n}):", file=out)
    for i in range(n):
        major, minor = torch.cuda.get_device_capability(i)
        ok = (major, minor) == (10, 0)
        print(f"  cuda:{i}  {torch.cuda.get_device_name(i)}  sm_{major}{minor}"
              f"{'' if ok else '   NOT IN THIS BUILD (sm_100a only)'}", file=out)
        rc |= 0 if ok else 1
    if n == 0:
        print("  none visible: only the CPU/gloo backend can run here", file=out)
    if n >= 2:
        matrix = fu.nvlink_matrix(range(n))
        if matrix is None:
            print("nvlink: NVML cannot say (the group constructor fails open)", file=out)
        else:
            print("nvlink (y = joined, N = not, . = self):", file=out)
            print("       " + " ".join(f"{j:>2}" for j in range(n)), file=out)
            for i in range(n):
                row = " ".join(" ." if i == j else (" y" if matrix[(i, j)] else " N") for j in range(n))
                print(f"  {i:>3}  {row}", file=out)
            if not all(matrix.values()):
                print("  some pairs are not NVLink-joined: UlyssesGroup(require_nvlink=True) will refuse them", file=out)
                rc |= 1
    return rc


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="fast_ulysses_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("doctor", help="report the build, the installed stack, the GPUs and their NVLink matrix")
    args = ap.parse_args(argv)
    if args.cmd == "doctor":
        return doctor()
    return 2


if __name__ == "__main__":
    sys.exit(main())
