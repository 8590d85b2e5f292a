"""Single-GPU tests of the all-to-all kernel and of the group runtime.

The multi-rank data path is exercised on ONE device by giving the kernel "peer" windows that are
ordinary buffers on the same device and running the ranks one after another with the handshakes
switched off (kernels that wait on one another must never run as separate launches on one GPU).
The oracle is a plain torch statement of the exchange on the global tensor."""

import ctypes as C

import pytest
import torch

import fast_ulysses_b200 as fu
from fast_ulysses_b200.ops import _ckernels as ck

pytestmark = pytest.mark.gpu
plan_debug = torch.ops.fast_ulysses_b200.a2a_plan_debug


def global_tensor(b, S, N, d, dtype, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype in (torch.int8, torch.uint8):
        return torch.randint(0, 120, (b, S, N, d), device="cuda", generator=g).to(dtype)
    x = torch.randn(b, S, N, d, device="cuda", generator=g)
    return x.to(dtype)


def shards(glob, seq, heads, mode):
    s0 = [sum(seq[:p]) for p in range(len(seq))]
    h0 = [sum(heads[:p]) for p in range(len(heads))]
    by_seq = [glob[:, s0[p]:s0[p] + seq[p]].contiguous() for p in range(len(seq))]
    by_head = [glob[:, :, h0[p]:h0[p] + heads[p]].contiguous() for p in range(len(seq))]
    return (by_seq, by_head) if mode == 0 else (by_head, by_seq)


def emulate(b, seq, heads, d, mode, dtype, flags, copy_out, ctas=0, own_direct=True):
    ws = len(seq)
    glob = global_tensor(b, sum(seq), sum(heads), d, dtype)
    inputs, expected = shards(glob, seq, heads, mode)
    elem = glob.element_size()
    plans = [plan_debug(b, d, r, ws, seq, heads, mode, elem) for r in range(ws)]
    wbytes = (plans[0][1] * elem + 255) // 256 * 256
    wins = [torch.zeros(wbytes + ck.FU_CTRL_BYTES, dtype=torch.uint8, device="cuda") for _ in range(ws)]
    outs = [torch.zeros(tuple(plans[r][0]), dtype=dtype, device="cuda") for r in range(ws)]
    stream = torch.cuda.current_stream().cuda_stream
    passes = [False, True] if copy_out else [False]
    # pass 1 pushes every rank's share; pass 2 (copy-out) runs again so that each rank's window is
    # complete before it is copied out -- re-pushing identical bytes is harmless
    for with_out in passes:
        for r in range(ws):
            a = ck.FuA2AArgs()
            a.src = inputs[r].data_ptr()
            for p in range(ws):
                a.peer_win[p] = wins[p].data_ptr()
                a.peer_ctrl[p] = wins[p].data_ptr() + wbytes
            a.rank, a.world = r, ws
            a.win_bytes, a.src_bytes = wbytes, inputs[r].numel() * elem
            a.flags = flags | ck.FU_A2A_NO_HANDSHAKE
            a.ctas = ctas
            rows = plans[r][2].tolist()
            a.n_routes = len(rows)
            for i, row in enumerate(rows):
                a.routes[i] = ck.route_from_row(row)
            if with_out:
                a.out = outs[r].data_ptr()
                a.out_bytes = outs[r].numel() * elem
                if own_direct:
                    a.own_direct = 1
                    keep = plans[r][4].tolist()
                    a.n_out_routes = len(keep)
                    for i, row in enumerate(keep):
                        a.out_routes[i] = ck.route_from_row(row)
            ck.check(ck.lib().fu_a2a4d(C.byref(a), C.c_void_p(stream)))
    torch.cuda.synchronize()
    for r in range(ws):
        n = expected[r].numel()
        got = wins[r][: n * elem].view(dtype).reshape(expected[r].shape)
        # pass 1 (no output tensor) filled the whole window, the own share included
        assert torch.equal(got.view(torch.uint8), expected[r].view(torch.uint8)), f"window of rank {r}"
        if copy_out:
            assert torch.equal(outs[r].view(torch.uint8), expected[r].view(torch.uint8)), f"copy-out of rank {r}"
        status = wins[r][wbytes + 80: wbytes + 84].view(torch.int32).item()
        assert status == 0, f"rank {r} status {status}"


@pytest.mark.parametrize("flags", [0, ck.FU_A2A_LDST, ck.FU_A2A_COPY_ENGINE], ids=["bulk", "ldst", "copy_engine"])
@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("ws", [1, 2, 3, 4, 8])
def test_even_shards(flags, mode, ws):
    emulate(2, [40] * ws, [2] * ws, 64, mode, torch.bfloat16, flags, copy_out=True)


@pytest.mark.parametrize("flags", [0, ck.FU_A2A_LDST, ck.FU_A2A_COPY_ENGINE], ids=["bulk", "ldst", "copy_engine"])
@pytest.mark.parametrize("mode", [0, 1])
def test_uneven_and_empty_shards(flags, mode):
    emulate(1, [300, 212], [4, 4], 128, mode, torch.float32, flags, copy_out=True)
    emulate(2, [17, 0, 33], [14, 13, 13], 128, mode, torch.bfloat16, flags, copy_out=True)
    emulate(1, [9, 1, 5, 2, 7, 11, 3], [1, 3, 2, 1, 4, 2, 5], 16, mode, torch.float16, flags, copy_out=False)


@pytest.mark.parametrize("dtype,d", [(torch.float32, 4), (torch.float16, 8), (torch.float8_e4m3fn, 16),
                                     (torch.float8_e5m2, 32), (torch.int8, 16), (torch.uint8, 48)])
def test_dtypes(dtype, d):
    for mode in (0, 1):
        emulate(2, [5, 9, 2], [3, 1, 2], d, mode, dtype, 0, copy_out=True)


@pytest.mark.parametrize("flags", [0, ck.FU_A2A_LDST, ck.FU_A2A_COPY_ENGINE], ids=["bulk", "ldst", "copy_engine"])
def test_flat_copy_out_without_own_direct(flags):
    emulate(2, [17, 5, 33], [2, 3, 1], 64, 0, torch.bfloat16, flags, copy_out=True, own_direct=False)
    emulate(2, [17, 5, 33], [2, 3, 1], 64, 1, torch.bfloat16, flags, copy_out=True, own_direct=False)


def test_rows_wider_than_a_stage_and_many_chunks():
    # one row = 40 heads x 512 x 4 B = 80 KiB > a 48 KiB stage: rows are split into pieces
    emulate(1, [37], [40], 512, 0, torch.float32, 0, copy_out=True)
    # many chunks per CTA with few CTAs exercises stage reuse and parity wrap
    emulate(1, [3000, 2900], [5, 5], 128, 0, torch.bfloat16, 0, copy_out=True, ctas=4)
    emulate(1, [3000, 2900], [5, 5], 128, 1, torch.bfloat16, 0, copy_out=True, ctas=2)


def test_group_single_rank_paths():
    g = fu.UlyssesGroup(device="cuda")
    x = torch.randn(2, 300, 8, 128, device="cuda", dtype=torch.bfloat16)
    y = g.all_to_all_4d(x)
    assert torch.equal(y, x) and y.data_ptr() != x.data_ptr()
    assert g._handle.epoch_debug(x, 0) == 2
    back = g.all_to_all_4d(y, mode=1)
    assert torch.equal(back, x)
    assert g._handle.epoch_debug(x, 0) == 4

    # zero-copy: the peers (here: this rank) write the caller's buffer directly
    out = g.empty_output(x)
    n_alloc = g._handle.windows_allocated()
    got = g.all_to_all_4d(x, out=out)
    assert got is out and torch.equal(out, x)
    assert g._handle.epoch_debug(out, 2) == 2 and g._handle.windows_allocated() == n_alloc
    assert g._handle.epoch_debug(x, 0) == 4  # the internal window was not involved

    # a strided view is read in place
    packed = torch.randn(2, 300, 3, 8, 128, device="cuda", dtype=torch.bfloat16)
    q = packed[:, :, 1]
    assert not q.is_contiguous()
    assert torch.equal(g.all_to_all_4d(q), q)

    # async, lent windows rotate through four slots
    h = g.all_to_all_4d_async(x)
    assert torch.equal(h.wait(), x)
    lent = [g.all_to_all_4d_async(x, lend=True).wait() for _ in range(4)]
    assert len({t.data_ptr() for t in lent}) == 4 and all(torch.equal(t, x) for t in lent)
    with pytest.raises(RuntimeError, match="lent results may be alive at once"):
        g.all_to_all_4d_async(x, lend=True)
    del lent
    again = g.all_to_all_4d_async(x, lend=True).wait()
    assert torch.equal(again, x)

    # the kernel's own phase timing
    _, stages = g._timed(x)
    assert set(stages) == {"barrier_in", "transfer", "barrier_out", "copy_out"}
    assert all(v >= 0 for v in stages.values()) and stages["transfer"] > 0

    # autograd on device
    xg = x.float().requires_grad_()
    yg = g.all_to_all_4d(xg)
    yg.square().sum().backward()
    assert torch.allclose(xg.grad, 2 * xg.detach())
    g.check()
    g.destroy()
    with pytest.raises(RuntimeError, match="has been destroyed"):
        g.all_to_all_4d(x)


@pytest.mark.parametrize("flags", [0, ck.FU_A2A_LDST], ids=["bulk", "ldst"])
@pytest.mark.parametrize("mode", [0, 1])
def test_pool_buffers_chosen_rank_by_rank(flags, mode):
    """Emulated ranks, each with its own choice of destination: its window, or one of two pool buffers.
    Every sender must follow every receiver's choice."""
    b, d, dtype = 2, 64, torch.bfloat16
    seq, heads = [40, 33, 0, 52, 17], [2, 3, 1, 2, 2]
    ws = len(seq)
    slots = [1, 0, 2, 2, 1]
    glob = global_tensor(b, sum(seq), sum(heads), d, dtype)
    inputs, expected = shards(glob, seq, heads, mode)
    elem = glob.element_size()
    plans = [plan_debug(b, d, r, ws, seq, heads, mode, elem) for r in range(ws)]
    wbytes = (plans[0][1] * elem + 255) // 256 * 256
    wins = [torch.zeros(wbytes + ck.FU_CTRL_BYTES, dtype=torch.uint8, device="cuda") for _ in range(ws)]
    pools = [[torch.zeros(wbytes, dtype=torch.uint8, device="cuda") for _ in range(2)] for _ in range(ws)]
    stream = torch.cuda.current_stream().cuda_stream
    for r in range(ws):
        a = ck.FuA2AArgs()
        a.src = inputs[r].data_ptr()
        for p in range(ws):
            a.peer_win[p] = wins[p].data_ptr()
            a.peer_ctrl[p] = wins[p].data_ptr() + wbytes
            a.peer_slot[p] = slots[p]
            for k in range(2):
                a.peer_pool[p][k] = pools[p][k].data_ptr()
        a.n_pool, a.my_slot = 2, slots[r]
        a.rank, a.world = r, ws
        a.win_bytes, a.pool_bytes, a.src_bytes = wbytes, wbytes, inputs[r].numel() * elem
        a.flags = flags | ck.FU_A2A_NO_HANDSHAKE
        rows = plans[r][2].tolist()
        a.n_routes = len(rows)
        for i, row in enumerate(rows):
            a.routes[i] = ck.route_from_row(row)
        if slots[r] > 0:  # the own share goes straight into the chosen buffer, nothing is copied out
            a.out = pools[r][slots[r] - 1].data_ptr()
            a.out_bytes = expected[r].numel() * elem
            a.own_direct = 1
        ck.check(ck.lib().fu_a2a4d(C.byref(a), C.c_void_p(stream)))
    torch.cuda.synchronize()
    for r in range(ws):
        n = expected[r].numel() * elem
        where = wins[r] if slots[r] == 0 else pools[r][slots[r] - 1]
        assert torch.equal(where[:n], expected[r].contiguous().view(torch.uint8).reshape(-1)), f"rank {r}"
        for k in range(2):
            if k != slots[r] - 1:
                assert not pools[r][k].any(), f"rank {r}: buffer {k} was not chosen but was written"
    # a choice that does not exist is refused on the host
    a.my_slot = 3
    assert ck.lib().fu_a2a4d(C.byref(a), C.c_void_p(stream)) != 0


def test_output_pool_of_the_copying_call():
    g = fu.UlyssesGroup(device="cuda")
    h = g._handle
    assert h.output_pool()
    x = torch.randn(2, 300, 8, 128, device="cuda", dtype=torch.bfloat16)
    held = [g.all_to_all_4d(x) for _ in range(3)]
    assert h.pool_hits() == 3 and len({t.data_ptr() for t in held}) == 3
    n_alloc = h.windows_allocated()
    extra = g.all_to_all_4d(x)  # every buffer is referenced: this call goes through the window
    assert h.pool_hits() == 3 and torch.equal(extra, x) and extra.data_ptr() not in {t.data_ptr() for t in held}
    first = held[0].data_ptr()
    view = held[0][:, :10]  # a view keeps the buffer alive
    del held[0]
    y = g.all_to_all_4d(x)
    assert h.pool_hits() == 3 and torch.equal(view, x[:, :10])
    del view, y
    y = g.all_to_all_4d(x)
    assert h.pool_hits() == 4 and y.data_ptr() == first and h.windows_allocated() == n_alloc
    assert all(torch.equal(t, x) for t in held)
    # a larger call replaces the pool; results handed out before stay valid
    big = torch.randn(2, 700, 8, 128, device="cuda", dtype=torch.bfloat16)
    yb = g.all_to_all_4d(big)
    assert torch.equal(yb, big) and h.windows_allocated() > n_alloc and all(torch.equal(t, x) for t in held)
    # a buffer filled on one stream and taken again on another: the second call waits for what
    # was queued on the first (here a slow reader of the dropped result)
    side = torch.cuda.Stream()
    tmp = g.all_to_all_4d(x)
    acc = torch.zeros_like(tmp, dtype=torch.float32)
    for _ in range(50):
        acc += tmp.float()
    del tmp
    side.wait_stream(torch.cuda.current_stream())
    other = torch.randn_like(x)
    with torch.cuda.stream(side):
        outs = [g.all_to_all_4d(other) for _ in range(4)]
    torch.cuda.synchronize()
    assert torch.allclose(acc, 50 * x.float()) and all(torch.equal(t, other) for t in outs)
    del outs
    h.set_output_pool(False)
    hits = h.pool_hits()
    assert torch.equal(g.all_to_all_4d(x), x) and h.pool_hits() == hits
    g.check()
    g.destroy()
    assert torch.equal(y, x) and torch.equal(yb, big)  # the memory outlives the group


def test_cuda_graph_replay_advances_epoch():
    g = fu.UlyssesGroup(device="cuda")
    x = torch.randn(1, 512, 8, 128, device="cuda", dtype=torch.bfloat16)
    out = g.empty_output(x)
    g.all_to_all_4d(x, out=out)  # warm: plan and window exist before capture
    torch.cuda.synchronize()
    e0 = g._handle.epoch_debug(out, 2)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        g.all_to_all_4d(x, out=out)
    for i in range(5):
        x.fill_(float(i))
        graph.replay()
        torch.cuda.synchronize()
        assert torch.all(out == float(i))
    # capture does not execute; five replays, two phases each
    assert g._handle.epoch_debug(out, 2) == e0 + 10
    # the copying call inside a capture: the result must not come out of the output pool, whose
    # buffers go back to other callers while the graph is still replayed
    y0 = g.all_to_all_4d(x)  # warm: window and pool exist
    hits = g._handle.pool_hits()
    torch.cuda.synchronize()
    graph2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph2):
        y = g.all_to_all_4d(x)
    assert g._handle.pool_hits() == hits
    for i in range(3):
        x.fill_(float(10 + i))
        graph2.replay()
        torch.cuda.synchronize()
        assert torch.all(y == float(10 + i))
    del y0
    g.destroy()


def test_wait_runs_out_and_reports():
    """A flag that nothing sets: a 2-rank group emulated with a mute peer. The wait ends by itself
    after the limit, the kernel returns, the status words say who was missing."""
    ws, b, d, elem = 2, 1, 16, 2
    seq, heads = [8, 8], [1, 1]
    plans = plan_debug(b, d, 0, ws, seq, heads, 0, elem)
    wbytes = 256 * ((plans[1] * elem + 255) // 256)
    wins = [torch.zeros(wbytes + ck.FU_CTRL_BYTES, dtype=torch.uint8, device="cuda") for _ in range(ws)]
    x = torch.zeros(b, 8, 2, d, dtype=torch.bfloat16, device="cuda")
    a = ck.FuA2AArgs()
    a.src = x.data_ptr()
    for p in range(ws):
        a.peer_win[p] = wins[p].data_ptr()
        a.peer_ctrl[p] = wins[p].data_ptr() + wbytes
    a.rank, a.world, a.timeout_ms = 0, ws, 200
    a.win_bytes, a.src_bytes = wbytes, x.numel() * elem
    rows = plans[2].tolist()
    a.n_routes = len(rows)
    for i, row in enumerate(rows):
        a.routes[i] = ck.route_from_row(row)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    ck.check(ck.lib().fu_a2a4d(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    t1.record()
    torch.cuda.synchronize()  # returns: the wait was bounded
    assert t0.elapsed_time(t1) < 5000
    status = wins[0][wbytes + 80: wbytes + 104].view(torch.int32).tolist()
    assert status[0] == 1 and status[1] == 1, status  # opening handshake, waiting on rank 1
    # the context is still usable
    assert torch.ones(4, device="cuda").sum().item() == 4
