"""ctypes view of ``lib/libfu_kernels.so``: the C structs of csrc/kernels/fu_kernels.h and a loader.

The torch operator layer (``_C.so``) links the same library; this module is the direct route used
by the fused operators in :mod:`fast_ulysses_b200.ops` and by kernel-level tests, which hand raw
device pointers to the launchers.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

FU_MAX_WORLD = 8
FU_POOL_SLOTS = 4
FU_CTRL_BYTES = 256

FU_A2A_NO_HANDSHAKE = 1
FU_A2A_STAMPS = 2
FU_A2A_EARLY_PUBLISH = 4
FU_A2A_LDST = 8
FU_A2A_COPY_ENGINE = 128
FU_A2A_MUTE = 16
FU_A2A_MINOR_SHARE = 32
FU_QKV_W_KN = 64


class FuRoute(C.Structure):
    _fields_ = [("peer", C.c_int32), ("pad_", C.c_int32), ("src_off", C.c_int64), ("dst_off", C.c_int64),
                ("src_pitch", C.c_int64), ("dst_pitch", C.c_int64), ("row_bytes", C.c_int64), ("rows", C.c_int64),
                ("batches", C.c_int64), ("src_batch", C.c_int64), ("dst_batch", C.c_int64)]


class FuA2AArgs(C.Structure):
    _fields_ = [("src", C.c_void_p), ("peer_win", C.c_void_p * FU_MAX_WORLD),
                ("peer_ctrl", C.c_void_p * FU_MAX_WORLD), ("out", C.c_void_p), ("out_bytes", C.c_int64),
                ("rank", C.c_int32), ("world", C.c_int32), ("n_routes", C.c_int32), ("flags", C.c_int32),
                ("ctas", C.c_int32), ("timeout_ms", C.c_uint32), ("routes", FuRoute * FU_MAX_WORLD),
                ("own_direct", C.c_int32), ("n_out_routes", C.c_int32), ("out_routes", FuRoute * 2),
                ("peer_pool", (C.c_void_p * FU_POOL_SLOTS) * FU_MAX_WORLD), ("n_pool", C.c_int32),
                ("my_slot", C.c_int32), ("peer_slot", C.c_int8 * FU_MAX_WORLD), ("win_bytes", C.c_int64),
                ("pool_bytes", C.c_int64), ("src_bytes", C.c_int64)]


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
        for name in ("fu_gemm_bf16", "fu_qkv_rope_scatter", "fu_fmha_fwd", "fu_fmha_bwd", "fu_pull_outproj",
                     "fu_qk_norm_rope_bwd"):
            getattr(_lib, name).restype = C.c_int
            getattr(_lib, name).argtypes = [C.c_void_p, C.c_void_p]
        _lib.fu_layernorm_fwd.restype = C.c_int
        _lib.fu_layernorm_fwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                          C.c_float, C.c_void_p]
        _lib.fu_layernorm_bwd.restype = C.c_int
        _lib.fu_layernorm_bwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                          C.c_void_p]
        _lib.fu_pull_qkv_grads.restype = C.c_int
        _lib.fu_pull_qkv_grads.argtypes = [C.c_void_p, C.c_void_p]
        _lib.fu_a2a4d_fp8.restype = C.c_int
        _lib.fu_a2a4d_fp8.argtypes = [C.c_void_p, C.c_void_p]
        for name in ("fu_a2a4d_check", "fu_qkv_rope_scatter_check", "fu_pull_outproj_check", "fu_pull_qkv_grads_check",
                     "fu_a2a4d_fp8_check"):
            getattr(_lib, name).restype = C.c_int
            getattr(_lib, name).argtypes = [C.c_void_p]
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(f"fast_ulysses_b200 kernel launch refused ({rc}): {lib().fu_last_error().decode()}")


def route_from_row(row) -> FuRoute:
    """A row of ``a2a_plan_debug``'s route tensor -> FuRoute."""
    peer, src_off, dst_off, src_pitch, dst_pitch, row_bytes, rows, batches, src_batch, dst_batch = (int(v) for v in row)
    return FuRoute(peer, 0, src_off, dst_off, src_pitch, dst_pitch, row_bytes, rows, batches, src_batch, dst_batch)


class FuGemmArgs(C.Structure):
    _fields_ = [("a", C.c_void_p), ("b", C.c_void_p), ("c", C.c_void_p), ("m", C.c_int64), ("n", C.c_int64),
                ("k", C.c_int64), ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64), ("bias", C.c_void_p),
                ("residual", C.c_void_p), ("act", C.c_int32), ("ctas", C.c_int32), ("err", C.c_void_p),
                ("flags", C.c_int32), ("aux", C.c_void_p), ("c_pre", C.c_void_p)]


class FuQkvArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("w", C.c_void_p), ("m", C.c_int64), ("k", C.c_int64), ("ldx", C.c_int64),
                ("ldw", C.c_int64), ("heads", C.c_int32), ("pad_", C.c_int32), ("s_local", C.c_int64),
                ("seq_off", C.c_int64), ("s_total", C.c_int64), ("rope", C.c_void_p), ("gamma_q", C.c_void_p),
                ("gamma_k", C.c_void_p), ("eps", C.c_float), ("rank", C.c_int32), ("world", C.c_int32),
                ("head_splits", C.c_int32 * FU_MAX_WORLD), ("win_q", C.c_void_p * FU_MAX_WORLD),
                ("win_k", C.c_void_p * FU_MAX_WORLD), ("win_v", C.c_void_p * FU_MAX_WORLD),
                ("peer_ctrl", C.c_void_p * FU_MAX_WORLD), ("flags", C.c_int32), ("timeout_ms", C.c_uint32),
                ("ctas", C.c_int32), ("err", C.c_void_p), ("n_types", C.c_int32), ("n_normed", C.c_int32),
                ("y_save", C.c_void_p), ("ld_y", C.c_int64), ("win_bytes", C.c_int64)]


def stream_ptr():
    import torch

    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class FuFmhaArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("lse", C.c_void_p),
                ("batch", C.c_int32), ("heads", C.c_int32), ("seq_q", C.c_int32), ("seq_kv", C.c_int32),
                ("head_dim", C.c_int32), ("scale", C.c_float),
                ("q_row", C.c_int64), ("q_head", C.c_int64), ("q_batch", C.c_int64),
                ("k_row", C.c_int64), ("k_head", C.c_int64), ("k_batch", C.c_int64),
                ("v_row", C.c_int64), ("v_head", C.c_int64), ("v_batch", C.c_int64),
                ("o_row", C.c_int64), ("o_head", C.c_int64), ("o_batch", C.c_int64),
                ("ctas", C.c_int32), ("flags", C.c_int32), ("err", C.c_void_p),
                ("d_o", C.c_void_p), ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
                ("delta", C.c_void_p), ("dq_acc", C.c_void_p), ("trace", C.c_void_p)]


class FuPullArgs(C.Structure):
    _fields_ = [("w", C.c_void_p), ("c", C.c_void_p), ("m", C.c_int64), ("n", C.c_int64), ("ldw", C.c_int64),
                ("ldc", C.c_int64), ("bias", C.c_void_p), ("residual", C.c_void_p), ("s_local", C.c_int64),
                ("seq_off", C.c_int64), ("s_total", C.c_int64), ("rank", C.c_int32), ("world", C.c_int32),
                ("head_splits", C.c_int32 * FU_MAX_WORLD), ("peer_o", C.c_void_p * FU_MAX_WORLD),
                ("peer_ctrl", C.c_void_p * FU_MAX_WORLD), ("gather", C.c_void_p), ("ready", C.c_void_p),
                ("flags", C.c_int32), ("timeout_ms", C.c_uint32), ("ctas", C.c_int32), ("pad_", C.c_int32),
                ("err", C.c_void_p), ("o_bytes", C.c_int64), ("gather_bytes", C.c_int64), ("ready_words", C.c_int64)]


class FuNormRopeBwdArgs(C.Structure):
    _fields_ = [("dq", C.c_void_p), ("dk", C.c_void_p), ("y", C.c_void_p), ("dy", C.c_void_p), ("rope", C.c_void_p),
                ("gamma_q", C.c_void_p), ("gamma_k", C.c_void_p), ("dgamma_q", C.c_void_p), ("dgamma_k", C.c_void_p),
                ("m", C.c_int64), ("s_local", C.c_int64), ("ld_y", C.c_int64), ("ld_dy", C.c_int64),
                ("heads", C.c_int32), ("eps", C.c_float)]


class FuPullGradsArgs(C.Structure):
    _fields_ = [("peer_dq", C.c_void_p * FU_MAX_WORLD), ("peer_dk", C.c_void_p * FU_MAX_WORLD),
                ("peer_dv", C.c_void_p * FU_MAX_WORLD), ("peer_ctrl", C.c_void_p * FU_MAX_WORLD),
                ("src_bytes", C.c_int64), ("y", C.c_void_p), ("dy", C.c_void_p), ("rope", C.c_void_p),
                ("gamma_q", C.c_void_p), ("gamma_k", C.c_void_p), ("dgamma_q", C.c_void_p), ("dgamma_k", C.c_void_p),
                ("m", C.c_int64), ("s_local", C.c_int64), ("seq_off", C.c_int64), ("s_total", C.c_int64),
                ("ld_y", C.c_int64), ("ld_dy", C.c_int64), ("heads", C.c_int32), ("rank", C.c_int32),
                ("world", C.c_int32), ("head_splits", C.c_int32 * FU_MAX_WORLD), ("flags", C.c_int32),
                ("timeout_ms", C.c_uint32), ("eps", C.c_float)]


class FuA2AFp8Args(C.Structure):
    _fields_ = [("src", C.c_void_p), ("out", C.c_void_p), ("peer_win", C.c_void_p * FU_MAX_WORLD),
                ("peer_ctrl", C.c_void_p * FU_MAX_WORLD), ("win_bytes", C.c_int64), ("src_bytes", C.c_int64),
                ("out_rows", C.c_int64), ("rank", C.c_int32), ("world", C.c_int32), ("n_routes", C.c_int32),
                ("flags", C.c_int32), ("ctas", C.c_int32), ("timeout_ms", C.c_uint32), ("routes", FuRoute * FU_MAX_WORLD)]
