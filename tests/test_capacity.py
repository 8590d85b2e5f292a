"""Every launcher that stores into, or loads from, another rank's memory checks on the host that
the last byte its address formula can reach lies inside the buffer it was given, and refuses the
launch otherwise. These checks make no CUDA call, so they are tested here without a GPU: the
arguments are built with made-up addresses that nothing ever dereferences."""

import ctypes as C

import pytest

from fast_ulysses_b200.ops import _ckernels as ck

BASE = 0x7F0000000000  # made-up, 16-byte aligned


def last_error() -> str:
    return ck.lib().fu_last_error().decode()


def a2a_args(world=2, rank=0, rows=8, row_bytes=256, win_bytes=8 * 256 * 2, src_bytes=8 * 512):
    """Rank `rank` of `world` sends `rows` rows of `row_bytes` to every rank; destination offset by sender."""
    a = ck.FuA2AArgs()
    a.src = BASE
    a.rank, a.world = rank, world
    a.win_bytes, a.src_bytes = win_bytes, src_bytes
    for p in range(world):
        a.peer_win[p] = BASE + (p + 1) * (1 << 30)
        a.peer_ctrl[p] = BASE + (p + 1) * (1 << 30) + win_bytes
        a.routes[p] = ck.FuRoute(p, 0, p * row_bytes, rank * rows * row_bytes, world * row_bytes, row_bytes, row_bytes, rows,
                                 1, 0, 0)
    a.n_routes = world
    return a


def test_a2a_routes_inside_their_buffers_pass():
    assert ck.lib().fu_a2a4d_check(C.byref(a2a_args())) == 0, last_error()


def test_a2a_route_past_the_window_is_refused():
    a = a2a_args(rank=1)  # rank 1's share is the last of the window
    a.routes[1].dst_off += 256  # one row too far into rank 1's window
    assert ck.lib().fu_a2a4d_check(C.byref(a)) != 0
    assert "window of 4096 bytes" in last_error() and "rank 1" in last_error()


def test_a2a_route_past_the_input_is_refused():
    a = a2a_args(src_bytes=8 * 512 - 16)
    assert ck.lib().fu_a2a4d_check(C.byref(a)) != 0
    assert "input of 4080 bytes" in last_error()


def test_a2a_route_past_a_pool_buffer_is_refused():
    a = a2a_args(rank=1)
    a.n_pool = 1
    a.pool_bytes = a.win_bytes - 256  # a peer may pick the pool buffer, which is smaller
    for p in range(2):
        a.peer_pool[p][0] = BASE + (8 + p) * (1 << 30)
    assert ck.lib().fu_a2a4d_check(C.byref(a)) != 0
    assert "pool buffers hold" in last_error()


def test_a2a_copy_engine_transport_refuses_the_output_pool():
    a = a2a_args()
    a.flags = 128  # FU_A2A_COPY_ENGINE
    assert ck.lib().fu_a2a4d_check(C.byref(a)) == 0, last_error()
    a.n_pool, a.pool_bytes = 1, a.win_bytes
    for p in range(2):
        a.peer_pool[p][0] = BASE + (8 + p) * (1 << 30)
    assert ck.lib().fu_a2a4d_check(C.byref(a)) != 0
    assert "copy-engine transport" in last_error()


def test_a2a_direct_own_share_past_the_output_is_refused():
    a = a2a_args()
    a.out, a.out_bytes, a.own_direct = BASE + (1 << 40), 8 * 256 * 2 - 256, 1
    assert ck.lib().fu_a2a4d_check(C.byref(a)) == 0, last_error()  # rank 0's share ends at byte 2048
    a.routes[0].dst_off = 8 * 256  # as if it were rank 1's share
    assert ck.lib().fu_a2a4d_check(C.byref(a)) != 0
    assert "output of" in last_error()


def test_a2a_copy_out_route_and_negative_strides_are_refused():
    a = a2a_args()
    a.out, a.out_bytes, a.own_direct = BASE + (1 << 40), 8 * 256 * 2, 1
    a.n_out_routes = 1
    a.out_routes[0] = ck.FuRoute(0, 0, 2048, 2048, 256, 256, 256, 9, 1, 0, 0)  # nine rows where eight fit
    assert ck.lib().fu_a2a4d_check(C.byref(a)) != 0
    assert "copy-out route 0" in last_error()
    b = a2a_args()
    b.routes[1].dst_pitch = -256
    assert ck.lib().fu_a2a4d_check(C.byref(b)) != 0
    assert "negative" in last_error()


def qkv_args(seq_off=100, s_local=50, s_total=150, head_splits=(3, 2), batches=2):
    q = ck.FuQkvArgs()
    q.x, q.w = BASE, BASE + (1 << 30)
    q.m, q.k, q.ldx, q.ldw = batches * s_local, 256, 256, 256
    q.heads = sum(head_splits)
    q.s_local, q.seq_off, q.s_total = s_local, seq_off, s_total
    q.rope = q.gamma_q = q.gamma_k = BASE + (2 << 30)
    q.rank, q.world = 0, len(head_splits)
    for p, h in enumerate(head_splits):
        q.head_splits[p] = h
        q.win_q[p] = q.win_k[p] = q.win_v[p] = q.peer_ctrl[p] = BASE + (4 + p) * (1 << 30)
    q.win_bytes = batches * s_total * max(head_splits) * 256
    return q


def test_qkv_scatter_inside_the_windows_passes():
    assert ck.lib().fu_qkv_rope_scatter_check(C.byref(qkv_args())) == 0, last_error()


def test_qkv_scatter_with_a_wrong_sequence_offset_is_refused():
    """A seq_off that puts the rows past the end of the sequence would store into whatever lies behind
    a peer's window."""
    assert ck.lib().fu_qkv_rope_scatter_check(C.byref(qkv_args(seq_off=101))) != 0
    assert "do not lie inside a sequence of 150" in last_error()


def test_qkv_scatter_into_windows_that_are_too_small_is_refused():
    q = qkv_args()
    q.win_bytes -= 256
    assert ck.lib().fu_qkv_rope_scatter_check(C.byref(q)) != 0
    assert "stores to rank 0 reach byte" in last_error()


def pull_args(seq_off=0, s_local=64, s_total=128, head_splits=(2, 2)):
    q = ck.FuPullArgs()
    heads = sum(head_splits)
    q.w, q.c, q.gather, q.ready = BASE, BASE + (1 << 30), BASE + (2 << 30), BASE + (3 << 30)
    q.m, q.n, q.ldw, q.ldc = s_local, 256, heads * 128, 256
    q.s_local, q.seq_off, q.s_total = s_local, seq_off, s_total
    q.rank, q.world = 0, len(head_splits)
    for p, h in enumerate(head_splits):
        q.head_splits[p] = h
        q.peer_o[p] = q.peer_ctrl[p] = BASE + (4 + p) * (1 << 30)
    q.o_bytes = s_total * max(head_splits) * 256
    q.gather_bytes = s_local * heads * 256
    q.ready_words = ((s_local + 127) // 128) * len(head_splits)
    return q


def test_pull_inside_the_buffers_passes():
    assert ck.lib().fu_pull_outproj_check(C.byref(pull_args())) == 0, last_error()


@pytest.mark.parametrize("field,text", [("o_bytes", "loads from rank"), ("gather_bytes", "gathered operand"),
                                        ("ready_words", "flags needed")])
def test_pull_with_a_buffer_that_is_too_small_is_refused(field, text):
    q = pull_args(seq_off=64)
    setattr(q, field, getattr(q, field) - 1)
    assert ck.lib().fu_pull_outproj_check(C.byref(q)) != 0
    assert text in last_error()


def test_pull_of_the_gradients_past_a_peer_buffer_is_refused():
    a = ck.FuPullGradsArgs()
    head_splits, s_local, s_total = (2, 3), 10, 30
    a.y = a.dy = a.rope = a.gamma_q = a.gamma_k = BASE
    a.m, a.s_local, a.seq_off, a.s_total, a.ld_y, a.ld_dy = s_local, s_local, 20, s_total, 1280, 1920
    a.heads, a.rank, a.world = sum(head_splits), 0, 2
    for p, h in enumerate(head_splits):
        a.head_splits[p] = h
        a.peer_dq[p] = a.peer_dk[p] = a.peer_dv[p] = a.peer_ctrl[p] = BASE + (p + 1) * (1 << 30)
    a.src_bytes = s_total * max(head_splits) * 256
    assert ck.lib().fu_pull_qkv_grads_check(C.byref(a)) == 0, last_error()
    a.src_bytes -= 256
    assert ck.lib().fu_pull_qkv_grads_check(C.byref(a)) != 0 and "loads from rank 1 reach byte" in last_error()
    a.src_bytes += 256
    a.seq_off = 21
    assert ck.lib().fu_pull_qkv_grads_check(C.byref(a)) != 0 and "do not lie inside a sequence of 30" in last_error()


def test_fp8_exchange_route_past_the_packed_window_is_refused():
    a = ck.FuA2AFp8Args()
    a.src, a.out = BASE, BASE + (1 << 40)
    a.rank, a.world, a.n_routes = 0, 2, 2
    rows, heads = 8, 2                      # 8 tokens x 2 heads per peer, rows of 256 bytes
    for p in range(2):
        a.peer_win[p] = a.peer_ctrl[p] = BASE + (p + 1) * (1 << 30)
        a.routes[p] = ck.FuRoute(p, 0, p * heads * 256, 0, 2 * heads * 256, heads * 256, heads * 256, rows, 1, 0, 0)
    a.src_bytes, a.out_rows = rows * 2 * heads * 256, 2 * rows * heads
    a.win_bytes = 2 * rows * heads * 144    # both ranks' shares, packed
    assert ck.lib().fu_a2a4d_fp8_check(C.byref(a)) == 0, last_error()
    a.routes[1].dst_off = 2 * rows * heads * 256 - 256  # the last row of the window, then seven more
    assert ck.lib().fu_a2a4d_fp8_check(C.byref(a)) != 0 and "window of" in last_error()
    a.routes[1].dst_off = 0
    a.routes[0].row_bytes = 384             # not whole 128-value rows
    assert ck.lib().fu_a2a4d_fp8_check(C.byref(a)) != 0 and "whole 128-value rows" in last_error()
