"""Explains why the native extension failed to import, by comparing what it was built against
with what is installed now. Parity: python/fast_ulysses/_diagnose.py:13-85 of the reference."""

from __future__ import annotations

import sys
from pathlib import Path


def build_facts() -> dict[str, str]:
    """What the in-tree build recorded: torch version, CUDA version and Python tag at build time."""
    meta = Path(__file__).resolve().parent.parent / "build" / "build_meta.txt"
    facts: dict[str, str] = {}
    if meta.exists():
        for line in meta.read_text().splitlines():
            if "=" in line:
                k, v = line.split("=", 1)
                facts[k.strip()] = v.strip()
    return facts


def live_facts() -> dict[str, str]:
    import torch

    return {
        "torch": torch.__version__,
        "cuda": str(torch.version.cuda),
        "python": f"{sys.version_info.major}.{sys.version_info.minor}",
    }


def verdict(error: str, built: dict[str, str], live: dict[str, str]) -> str:
    lines = []
    for key in ("torch", "cuda", "python"):
        if key in built and built[key] != live.get(key):
            lines.append(f"built against {key} {built[key]}, running {key} {live.get(key)}")
    if "undefined symbol" in error and not lines:
        lines.append("an undefined symbol usually means libtorch changed since the build")
    if "libcudart" in error or "libcuda" in error:
        lines.append("the CUDA runtime library could not be loaded; check the CUDA major version")
    if "libfu_kernels" in error:
        lines.append("the kernel library lib/libfu_kernels.so is missing; rebuild with "
                     "`python -m fast_ulysses_b200._build --force`")
    if not lines:
        lines.append("rebuild with `python -m fast_ulysses_b200._build --force`")
    return "; ".join(lines)


def explain(exc: BaseException) -> str:
    err = str(exc)
    return (f"fast_ulysses_b200: the native extension did not load: {err}\n  diagnosis: "
            f"{verdict(err, build_facts(), live_facts())}")
