"""The allocation-free attention backward, called through its exported C symbol.

Who needs it: callers that cannot obtain device memory at the call site (a CUDA graph being
recorded, a plugin inside an application that owns the allocator, a latency-critical loop). They
pass inputs and outputs only; the scratch lives inside the library. The test checks two calls in
a row against the ordinary entry point (which takes caller-provided scratch), and the size limit.
Collected last on purpose: a failure here cannot hide the result of any other test."""

import ctypes as C
import math

import pytest
import torch

from fast_ulysses_b200.ops import _ckernels as ck
from fast_ulysses_b200.ops import attention, gemm

pytestmark = pytest.mark.gpu


def _args(q, k, v, o, lse, d_o, dq, dk, dv):
    a = ck.FuFmhaArgs()
    attention._fill(a, q, k, v, o)
    a.lse = lse.data_ptr()
    a.scale = 1.0 / math.sqrt(128)
    a.d_o, a.dq, a.dk, a.dv = d_o.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    return a


def rel_err(got, want):
    return ((got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-12)).item()


def test_no_alloc_backward_matches_the_ordinary_entry_point_twice():
    lib = ck.lib()
    fn = lib.fu_fmha_bwd_noalloc
    fn.restype, fn.argtypes = C.c_int, [C.c_void_p, C.c_void_p]
    for call, (b, h, sq, skv) in enumerate([(1, 2, 300, 500), (2, 3, 640, 384)]):
        torch.manual_seed(100 + call)
        q = torch.randn(b, sq, h, 128, device="cuda").bfloat16()
        k = torch.randn(b, skv, h, 128, device="cuda").bfloat16()
        v = torch.randn(b, skv, h, 128, device="cuda").bfloat16()
        o, lse = attention.fmha_fwd(q, k, v)
        d_o = torch.randn_like(o)
        want = attention.fmha_bwd(q, k, v, o, lse, d_o)  # existing entry point, torch-allocated scratch
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        a = _args(q, k, v, o, lse, d_o, dq, dk, dv)  # no scratch pointers at all
        before = torch.cuda.memory_allocated()
        ck.check(fn(C.byref(a), ck.stream_ptr()))
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        gemm.check_errors()
        # dK and dV are deterministic; dQ is summed by floating-point reductions in arbitrary order
        assert torch.equal(dk, want[1]) and torch.equal(dv, want[2]), f"call {call}"
        assert rel_err(dq, want[0]) < 2e-2, (call, rel_err(dq, want[0]))


def test_no_alloc_backward_refuses_what_does_not_fit():
    lib = ck.lib()
    fn = lib.fu_fmha_bwd_noalloc
    fn.restype, fn.argtypes = C.c_int, [C.c_void_p, C.c_void_p]
    q = torch.empty(1, 20000, 1, 128, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(1, 1, 20000, device="cuda")
    a = _args(q, q, q, q, lse, q, q, q, q)
    rc = fn(C.byref(a), ck.stream_ptr())
    assert rc != 0 and b"16384" in lib.fu_last_error()
    # the second limit: statistics are padded to 128 rows per (batch, head), so 1024 heads of one
    # row each (1024 rows, far below the first limit) do not fit either, and the message says which
    q = torch.empty(1, 1, 1024, 128, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(1, 1024, 1, device="cuda")
    a = _args(q, q, q, q, lse, q, q, q, q)
    rc = fn(C.byref(a), ck.stream_ptr())
    assert rc != 0 and b"65536" in lib.fu_last_error() and b"roundup" in lib.fu_last_error()
