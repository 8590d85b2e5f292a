"""Host-only tests of the layout contract: every rank's plan is replayed over plain numpy byte
buffers (one "window" per simulated rank) and compared with a numpy statement of the exchange.
Cases follow the reference's test/test_plan.py:151-333; nothing here needs a GPU or a process group.
"""

import numpy as np
import pytest
import torch

import fast_ulysses_b200  # noqa: F401

plan_debug = torch.ops.fast_ulysses_b200.a2a_plan_debug
COLS = ("peer", "src_off", "dst_off", "src_pitch", "dst_pitch", "row_bytes", "rows", "batches", "src_batch",
        "dst_batch")


def routes(t):
    return [dict(zip(COLS, (int(v) for v in row))) for row in t.tolist()]


def make_inputs(b, seq, heads, d, mode, dtype, seed=0):
    """Per-rank inputs carved out of one global (b, S, N, d) array."""
    rng = np.random.default_rng(seed)
    S, N = sum(seq), sum(heads)
    if np.issubdtype(dtype, np.floating):
        glob = rng.standard_normal((b, S, N, d)).astype(dtype)
    else:
        glob = rng.integers(0, 100, size=(b, S, N, d)).astype(dtype)
    s0 = np.concatenate([[0], np.cumsum(seq)])
    h0 = np.concatenate([[0], np.cumsum(heads)])
    ws = len(seq)
    seq_shards = [np.ascontiguousarray(glob[:, s0[r]:s0[r + 1]]) for r in range(ws)]
    head_shards = [np.ascontiguousarray(glob[:, :, h0[r]:h0[r + 1]]) for r in range(ws)]
    return (seq_shards, head_shards) if mode == 0 else (head_shards, seq_shards)


def replay(b, seq, heads, d, mode, inputs):
    """Run every rank's `sends` into per-rank byte windows; return each rank's output array."""
    ws = len(seq)
    elem = inputs[0].dtype.itemsize
    plans = [plan_debug(b, d, r, ws, list(seq), list(heads), mode, elem) for r in range(ws)]
    numel = {p[1] for p in plans}
    assert len(numel) == 1, "window_numel must be identical on every rank"
    wn = numel.pop()
    windows = [np.zeros(wn * elem, dtype=np.uint8) for _ in range(ws)]
    for r in range(ws):
        src = inputs[r].reshape(-1).view(np.uint8)
        for op in routes(plans[r][2]):
            dst = windows[op["peer"]]
            for bi in range(op["batches"]):
                for row in range(op["rows"]):
                    so = op["src_off"] + bi * op["src_batch"] + row * op["src_pitch"]
                    do = op["dst_off"] + bi * op["dst_batch"] + row * op["dst_pitch"]
                    dst[do:do + op["row_bytes"]] = src[so:so + op["row_bytes"]]
    outs = []
    for r in range(ws):
        shape = list(plans[r][0])
        n = int(np.prod(shape))
        assert n <= wn
        outs.append(windows[r][: n * elem].view(inputs[0].dtype).reshape(shape))
    return outs, plans


def check(b, seq, heads, d, mode, dtype=np.float32):
    inputs, expected = make_inputs(b, seq, heads, d, mode, dtype)
    outs, plans = replay(b, seq, heads, d, mode, inputs)
    for r, (got, want) in enumerate(zip(outs, expected)):
        assert got.shape == want.shape, (r, got.shape, want.shape)
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), f"rank {r} mismatch"
    return plans


@pytest.mark.parametrize("ws", [1, 2, 4, 8])
@pytest.mark.parametrize("b", [1, 3])
@pytest.mark.parametrize("mode", [0, 1])
def test_even(ws, b, mode):
    check(b, [6] * ws, [2] * ws, 8, mode)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("seq,heads", [
    ([5, 7, 3], [2, 2, 2]),
    ([4, 4, 4], [3, 1, 2]),
    ([300, 212], [4, 4]),
    ([9, 1, 5, 2, 7], [1, 3, 2, 1, 4]),
    ([14, 13, 13], [14, 13, 13]),
])
def test_uneven(mode, seq, heads):
    check(2, seq, heads, 4, mode)


@pytest.mark.parametrize("mode", [0, 1])
def test_empty_shard(mode):
    check(1, [4, 0, 3], [2, 1, 0], 4, mode)


@pytest.mark.parametrize("dtype,d", [(np.float16, 8), (np.float32, 4), (np.int8, 16), (np.uint8, 16)])
def test_dtypes(dtype, d):
    check(2, [3, 5], [2, 1], d, 0, dtype)
    check(2, [3, 5], [2, 1], d, 1, dtype)


def test_round_trip():
    b, seq, heads, d = 2, [5, 2, 6], [1, 3, 2], 4
    inputs, _ = make_inputs(b, seq, heads, d, 0, np.float32, seed=3)
    mid, _ = replay(b, seq, heads, d, 0, inputs)
    back, _ = replay(b, seq, heads, d, 1, [np.ascontiguousarray(m) for m in mid])
    for got, want in zip(back, inputs):
        assert np.array_equal(got, want)


def test_recvs_mirror_sends():
    b, seq, heads, d, elem = 2, [5, 2, 6], [1, 3, 2], 4, 2
    for mode in (0, 1):
        plans = [plan_debug(b, d, r, 3, seq, heads, mode, elem) for r in range(3)]
        for r in range(3):
            for rv in routes(plans[r][3]):
                match = [s for s in routes(plans[rv["peer"]][2]) if s["peer"] == r]
                assert len(match) == 1
                for k in ("dst_off", "dst_pitch", "row_bytes", "rows", "batches", "dst_batch"):
                    assert match[0][k] == rv[k]


def test_matches_torch_all_to_all_semantics():
    """Single-process statement of permute + all_to_all_single + permute for even shards."""
    ws, b, s_local, n, d = 4, 2, 3, 8, 4
    xs = [torch.randn(b, s_local, n, d) for _ in range(ws)]
    # what all_to_all_single would deliver: chunk r of rank p's (ws, b, s, n/ws, d) goes to rank r
    sent = [x.reshape(b, s_local, ws, n // ws, d).permute(2, 0, 1, 3, 4).contiguous() for x in xs]
    want = []
    for r in range(ws):
        recv = torch.stack([sent[p][r] for p in range(ws)])  # (ws, b, s, n/ws, d)
        want.append(recv.permute(1, 0, 2, 3, 4).reshape(b, ws * s_local, n // ws, d))
    outs, _ = replay(b, [s_local] * ws, [n // ws] * ws, d, 0, [x.numpy() for x in xs])
    for got, w in zip(outs, want):
        assert np.array_equal(got, w.numpy())


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("seq,heads", [([5, 7, 3], [3, 1, 2]), ([4, 0, 6], [2, 2, 0]), ([6], [3])])
def test_own_share_direct_plus_from_peers_covers_the_output(mode, seq, heads):
    """The copying call: own share straight to the output, `from_peers` regions copied out of the
    window. Together they must produce exactly the full output, and must not overlap."""
    b, d, dtype = 2, 4, np.float32
    ws = len(seq)
    inputs, expected = make_inputs(b, seq, heads, d, mode, dtype, seed=5)
    outs_win, plans = replay(b, seq, heads, d, mode, inputs)
    elem = 4
    for r in range(ws):
        want = expected[r]
        out = np.full(want.size * elem, 0xAB, dtype=np.uint8)
        written = np.zeros(want.size * elem, dtype=np.int32)
        src = inputs[r].reshape(-1).view(np.uint8)
        win = outs_win[r].reshape(-1).view(np.uint8)
        for op in routes(plans[r][2]):
            if op["peer"] != r:
                continue
            for bi in range(op["batches"]):
                for row in range(op["rows"]):
                    so = op["src_off"] + bi * op["src_batch"] + row * op["src_pitch"]
                    do = op["dst_off"] + bi * op["dst_batch"] + row * op["dst_pitch"]
                    out[do:do + op["row_bytes"]] = src[so:so + op["row_bytes"]]
                    written[do:do + op["row_bytes"]] += 1
        regions = routes(plans[r][4])
        assert len(regions) <= 2
        for op in regions:
            assert op["src_off"] == op["dst_off"] and op["src_pitch"] == op["dst_pitch"]
            for bi in range(op["batches"]):
                for row in range(op["rows"]):
                    o = op["src_off"] + bi * op["src_batch"] + row * op["src_pitch"]
                    out[o:o + op["row_bytes"]] = win[o:o + op["row_bytes"]]
                    written[o:o + op["row_bytes"]] += 1
        assert np.all(written == 1), f"rank {r}: every output byte written exactly once"
        assert np.array_equal(out, want.reshape(-1).view(np.uint8))


def test_window_numel_is_max_over_ranks():
    seq, heads = [5, 7, 3], [3, 1, 2]
    for mode in (0, 1):
        plans = [plan_debug(1, 4, r, 3, seq, heads, mode, 2) for r in range(3)]
        biggest = max(int(np.prod(list(p[0]))) for p in plans)
        assert all(p[1] == biggest for p in plans)


@pytest.mark.parametrize("kwargs,fragment", [
    (dict(seq=[1, 2], heads=[1, 1, 1]), "seq_splits has"),
    (dict(seq=[1, 2, 3], heads=[1, 1]), "head_splits has"),
    (dict(seq=[1, -2, 3], heads=[1, 1, 1]), "negative"),
    (dict(seq=[1, 2, 3], heads=[1, -1, 1]), "negative"),
    (dict(seq=[1, 2, 3], heads=[1, 1, 1], mode=2), "mode must be"),
    (dict(seq=[2 ** 40, 2 ** 40, 1], heads=[2 ** 20, 1, 1]), "overflows int64"),
])
def test_rejections(kwargs, fragment):
    mode = kwargs.pop("mode", 0)
    with pytest.raises(RuntimeError, match=fragment):
        plan_debug(1, 4, 0, 3, kwargs["seq"], kwargs["heads"], mode, 2)


# ---- property-based: any world size, any split, both modes ---------------------------------------------
hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402


@st.composite
def layouts(draw):
    ws = draw(st.integers(1, 8))
    seq = draw(st.lists(st.integers(0, 9), min_size=ws, max_size=ws))
    heads = draw(st.lists(st.integers(0, 5), min_size=ws, max_size=ws))
    if sum(seq) == 0:
        seq[draw(st.integers(0, ws - 1))] = 1 + draw(st.integers(0, 5))
    if sum(heads) == 0:
        heads[draw(st.integers(0, ws - 1))] = 1 + draw(st.integers(0, 3))
    return dict(b=draw(st.integers(1, 3)), seq=seq, heads=heads, d=draw(st.sampled_from([4, 8, 16, 32])),
                mode=draw(st.integers(0, 1)))


@settings(max_examples=60, deadline=None)
@given(layouts())
def test_any_layout_replays_to_the_permutation(lay):
    """Random world sizes and splits, empty shards included: replaying every rank's routes over byte
    windows gives exactly the exchange, the routes of all senders never overlap inside a window,
    and what lands in a window stays inside the uniform window size."""
    b, seq, heads, d, mode = lay["b"], lay["seq"], lay["heads"], lay["d"], lay["mode"]
    plans = check(b, seq, heads, d, mode, np.float32)
    ws, elem = len(seq), 4
    wn = plans[0][1]
    for target in range(ws):
        covered = np.zeros(wn * elem, dtype=np.uint8)
        for r in range(ws):
            for op in routes(plans[r][2]):
                if op["peer"] != target:
                    continue
                for bi in range(op["batches"]):
                    for row in range(op["rows"]):
                        do = op["dst_off"] + bi * op["dst_batch"] + row * op["dst_pitch"]
                        assert do + op["row_bytes"] <= wn * elem
                        assert not covered[do:do + op["row_bytes"]].any(), "two senders write the same bytes"
                        covered[do:do + op["row_bytes"]] = 1
        out_bytes = int(np.prod(list(plans[target][0]))) * elem
        assert covered[:out_bytes].all() and not covered[out_bytes:].any()


@settings(max_examples=40, deadline=None)
@given(layouts())
def test_mode_1_undoes_mode_0_for_any_layout(lay):
    b, seq, heads, d = lay["b"], lay["seq"], lay["heads"], lay["d"]
    inputs, _ = make_inputs(b, seq, heads, d, 0, np.float32, seed=3)
    mid, _ = replay(b, seq, heads, d, 0, inputs)
    back, _ = replay(b, seq, heads, d, 1, [np.ascontiguousarray(m) for m in mid])
    for r in range(len(seq)):
        assert np.array_equal(back[r], inputs[r])
