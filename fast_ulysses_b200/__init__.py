"""fast_ulysses_b200: a Blackwell-native Ulysses sequence-parallel library.

The public surface mirrors triple-mu/fast-ulysses (python/fast_ulysses/__init__.py:3-18):
``UlyssesGroup``, ``CompletedHandle``, ``nvlink_matrix`` and ``__version__``; on top of it come the
fused sm_100a operators in :mod:`fast_ulysses_b200.ops` and the sequence-parallel DiT blocks in
:mod:`fast_ulysses_b200.models`.
"""

from __future__ import annotations

import torch  # noqa: F401  (libtorch must be loaded before the extension)

__version__ = "0.1.0"


def _load_extension():
    from pathlib import Path

    pkg = Path(__file__).resolve().parent
    try:
        from . import _C  # type: ignore[attr-defined]
        return _C
    except ImportError as first:
        # Not built yet (a source checkout): build in-tree once, then import. A build that exists
        # but does not load is a different failure and is explained rather than rebuilt over.
        if (pkg / "_C.so").exists():
            from .utils.diagnose import explain

            raise ImportError(explain(first)) from first
        from . import _build

        _build.build_all(verbose=False)
        from . import _C  # type: ignore[attr-defined]
        return _C


_C = _load_extension()

from .parallel.group import CompletedHandle, UlyssesGroup  # noqa: E402


def nvlink_matrix(devices):
    """``{(i, j): joined by NVLink}`` for CUDA device indices, or ``None`` when NVML cannot say."""
    return _C.nvlink_matrix([int(d) for d in devices])


__all__ = ["UlyssesGroup", "CompletedHandle", "nvlink_matrix", "__version__"]
