"""ctypes view of ``lib/libfu_kernels.so``: the C structs of csrc/kernels/fu_kernels.h and a loader.

The torch operator layer (``_C.so``) links the same library; this module is the direct route used
by the fused operators in :mod:`fast_ulysses_b200.ops` and by kernel-level tests, which hand raw
device pointers to the launchers.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

FU_MAX_WORLD = 8
FU_CTRL_BYTES = 256

FU_A2A_NO_HANDSHAKE = 1
FU_A2A_STAMPS = 2
FU_A2A_EARLY_PUBLISH = 4
FU_A2A_LDST = 8
FU_A2A_MUTE = 16


class FuRoute(C.Structure):
    _fields_ = [("peer", C.c_int32), ("pad_", C.c_int32), ("src_off", C.c_int64), ("dst_off", C.c_int64),
                ("src_pitch", C.c_int64), ("dst_pitch", C.c_int64), ("row_bytes", C.c_int64), ("rows", C.c_int64),
                ("batches", C.c_int64), ("src_batch", C.c_int64), ("dst_batch", C.c_int64)]


class FuA2AArgs(C.Structure):
    _fields_ = [("src", C.c_void_p), ("peer_win", C.c_void_p * FU_MAX_WORLD),
                ("peer_ctrl", C.c_void_p * FU_MAX_WORLD), ("out", C.c_void_p), ("out_bytes", C.c_int64),
                ("rank", C.c_int32), ("world", C.c_int32), ("n_routes", C.c_int32), ("flags", C.c_int32),
                ("ctas", C.c_int32), ("timeout_ms", C.c_uint32), ("routes", FuRoute * FU_MAX_WORLD)]


_lib = None


def lib() -> C.CDLL:
    """Loads the kernel library (building it first if this is a fresh source checkout)."""
    global _lib
    if _lib is None:
        path = Path(__file__).resolve().parent.parent / "lib" / "libfu_kernels.so"
        if not path.exists():
            from .. import _build

            _build.build_kernels()
        _lib = C.CDLL(str(path))
        _lib.fu_last_error.restype = C.c_char_p
        _lib.fu_build_info.restype = C.c_char_p
        _lib.fu_a2a4d.argtypes = [C.POINTER(FuA2AArgs), C.c_void_p]
        _lib.fu_a2a4d.restype = C.c_int
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(f"fast_ulysses_b200 kernel launch refused ({rc}): {lib().fu_last_error().decode()}")


def route_from_row(row) -> FuRoute:
    """A row of ``a2a_plan_debug``'s route tensor -> FuRoute."""
    peer, src_off, dst_off, src_pitch, dst_pitch, row_bytes, rows, batches, src_batch, dst_batch = (int(v) for v in row)
    return FuRoute(peer, 0, src_off, dst_off, src_pitch, dst_pitch, row_bytes, rows, batches, src_batch, dst_batch)
