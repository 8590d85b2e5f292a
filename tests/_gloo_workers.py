"""Rank bodies for the CPU/gloo tests. Each takes (rank, world, ...) with the default group up."""

import torch
import torch.distributed as dist

from fast_ulysses_b200 import UlyssesGroup


def reference_uneven(x, mode, seq, heads, rank, world):
    """permute + all_to_all (list form) + permute, the torch.distributed statement of the exchange."""
    b, d = x.shape[0], x.shape[3]
    if mode == 0:
        h0 = [sum(heads[:p]) for p in range(world)]
        send = [x[:, :, h0[p]:h0[p] + heads[p]].contiguous() for p in range(world)]
        recv = [torch.empty(b, seq[p], heads[rank], d, dtype=x.dtype) for p in range(world)]
        _a2a_list(recv, send)
        return torch.cat(recv, dim=1)
    s0 = [sum(seq[:p]) for p in range(world)]
    send = [x[:, s0[p]:s0[p] + seq[p]].contiguous() for p in range(world)]
    recv = [torch.empty(b, seq[rank], heads[p], d, dtype=x.dtype) for p in range(world)]
    _a2a_list(recv, send)
    return torch.cat(recv, dim=2)


def _a2a_list(recv, send):
    """gloo has no list all_to_all; emulate it with all_to_all_single on flattened bytes."""
    flat_send = torch.cat([t.reshape(-1).view(torch.uint8) for t in send])
    in_sizes = [t.numel() * t.element_size() for t in send]
    out_sizes = [t.numel() * t.element_size() for t in recv]
    flat_recv = torch.empty(sum(out_sizes), dtype=torch.uint8)
    dist.all_to_all_single(flat_recv, flat_send, out_sizes, in_sizes)
    off = 0
    for t, n in zip(recv, out_sizes):
        t.copy_(flat_recv[off:off + n].view(t.dtype).reshape(t.shape))
        off += n


def reference_even(x, mode, world):
    """The baseline every Ulysses implementation ships: permute, all_to_all_single, permute."""
    b, s, n, d = x.shape
    if mode == 0:
        t = x.reshape(b, s, world, n // world, d).permute(2, 0, 1, 3, 4).contiguous()
        o = torch.empty_like(t)
        dist.all_to_all_single(o, t)
        return o.permute(1, 0, 2, 3, 4).reshape(b, world * s, n // world, d)
    t = x.reshape(b, world, s // world, n, d).permute(1, 0, 2, 3, 4).contiguous()
    o = torch.empty_like(t)
    dist.all_to_all_single(o, t)
    return o.permute(1, 2, 0, 3, 4).reshape(b, s // world, world * n, d)


def round_trip_config1(rank, world):
    """fp32 randn(seed), heads = 4*ws, d = 128, seq_splits [300, 212], even head splits: mode 0
    bitwise equal to the torch.distributed form, then mode 1 back to the input."""
    g = UlyssesGroup(device="cpu")
    seq = [300, 212][:world] if world == 2 else [300 - 7 * p for p in range(world)]
    heads = [4] * world
    torch.manual_seed(1234 + rank)
    x = torch.randn(1, seq[rank], 4 * world, 128)
    y = g.all_to_all_4d(x, mode=0, seq_splits=seq, head_splits=heads)
    want = reference_uneven(x, 0, seq, heads, rank, world)
    assert y.shape == (1, sum(seq), 4, 128)
    assert torch.equal(y, want)
    back = g.all_to_all_4d(y, mode=1, seq_splits=seq, head_splits=heads)
    assert torch.equal(back, x)
    g.destroy()


def even_and_dtypes(rank, world):
    g = UlyssesGroup(device="cpu")
    for dtype, d in [(torch.float32, 8), (torch.bfloat16, 8), (torch.float16, 16), (torch.int8, 16),
                     (torch.uint8, 32), (torch.float8_e4m3fn, 16)]:
        for mode in (0, 1):
            torch.manual_seed(7 + rank)
            shape = (2, 6, 2 * world, d) if mode == 0 else (2, 6 * world, 2, d)
            x = torch.randn(shape).mul(10).to(dtype) if dtype.is_floating_point else torch.randint(
                0, 100, shape).to(dtype)
            y = g.all_to_all_4d(x, mode=mode)
            xb, = (x.view(torch.uint8),)
            want = reference_even(xb, mode, world).view(dtype)
            assert torch.equal(y.view(torch.uint8), want.view(torch.uint8)), (dtype, mode)
    # out= variant and a non-contiguous input
    x = torch.randn(1, 4, 2 * world, 8)
    out = torch.empty(1, 4 * world, 2, 8)
    got = g.all_to_all_4d(x, out=out)
    assert got is out and torch.equal(out, reference_even(x, 0, world))
    xt = torch.randn(1, 2 * world, 4, 8).transpose(1, 2)
    assert torch.equal(g.all_to_all_4d(xt), reference_even(xt.contiguous(), 0, world))
    h = g.all_to_all_4d_async(x)
    assert torch.equal(h.wait(), reference_even(x, 0, world))
    g.destroy()


def autograd_paths(rank, world):
    g = UlyssesGroup(device="cpu")
    seq = [3 + p for p in range(world)]
    heads = [1 + (p % 2) for p in range(world)]
    torch.manual_seed(rank)
    x = torch.randn(2, seq[rank], sum(heads), 4, requires_grad=True)
    y = g.all_to_all_4d(x, mode=0, seq_splits=seq, head_splits=heads)
    w = torch.randn_like(y)
    (y * w).sum().backward()
    # backward == forward of the other mode with the same (unswapped) splits
    want = g.all_to_all_4d(w, mode=1, seq_splits=seq, head_splits=heads)
    assert torch.equal(x.grad, want)

    # double backward
    x2 = torch.randn(2, seq[rank], sum(heads), 4, requires_grad=True)
    y2 = g.all_to_all_4d(x2, mode=0, seq_splits=seq, head_splits=heads)
    (gx,) = torch.autograd.grad((y2 * y2).sum(), x2, create_graph=True)
    gx.sum().backward()
    assert torch.allclose(x2.grad, torch.full_like(x2, 2.0))

    # forward-mode AD: the tangent takes the same trip
    import torch.autograd.forward_ad as fwAD

    p = torch.randn(2, seq[rank], sum(heads), 4)
    t = torch.randn_like(p)
    with fwAD.dual_level():
        out = g.all_to_all_4d(fwAD.make_dual(p, t), mode=0, seq_splits=seq, head_splits=heads)
        primal, tangent = fwAD.unpack_dual(out)
    assert torch.equal(primal, g.all_to_all_4d(p, mode=0, seq_splits=seq, head_splits=heads))
    assert torch.equal(tangent, g.all_to_all_4d(t, mode=0, seq_splits=seq, head_splits=heads))

    # refusals that live in Python
    import pytest

    with pytest.raises(RuntimeError, match="does not support autograd"):
        g.all_to_all_4d(x, out=torch.empty(2, sum(seq), heads[rank], 4), seq_splits=seq, head_splits=heads)
    with pytest.raises(RuntimeError, match="does not support autograd"):
        g.all_to_all_4d_async(x, seq_splits=seq, head_splits=heads)
    with pytest.raises(ValueError, match="not both"):
        g.all_to_all_4d_async(x.detach(), out=torch.empty(1), lend=True)
    g.destroy()


def validation(rank, world):
    """Every rejection raises on every rank before anything collective happens; a rejection that
    were not uniform would leave the barrier after each case waiting for ever (the test's timeout)."""
    import pytest

    g = UlyssesGroup(device="cpu")
    ok = torch.randn(1, 4, 2 * world, 8)

    def rejects(fragment, fn, exc=RuntimeError):
        with pytest.raises(exc, match=fragment):
            fn()
        dist.barrier()

    rejects("must be 4D", lambda: g.all_to_all_4d(torch.randn(4, 2 * world, 8)))
    rejects("dtype must be", lambda: g.all_to_all_4d(ok.double()))
    rejects("dtype must be", lambda: g.all_to_all_4d(ok.int()))
    rejects("16-byte aligned", lambda: g.all_to_all_4d(torch.randn(1, 4, 2 * world, 4).bfloat16()))
    rejects("16-byte aligned", lambda: g.all_to_all_4d(torch.zeros(1, 4, 2 * world, 8, dtype=torch.int8)))
    rejects("mode must be 0 or 1", lambda: g.all_to_all_4d(ok, mode=2))
    rejects("both seq_splits and head_splits", lambda: g.all_to_all_4d(ok, seq_splits=[4] * world))
    rejects("but the splits imply",
            lambda: g.all_to_all_4d(ok, seq_splits=[5] * world, head_splits=[2] * world))
    rejects("must divide world_size", lambda: g.all_to_all_4d(torch.randn(1, 4, 2 * world + 1, 8)))
    rejects("must divide world_size", lambda: g.all_to_all_4d(torch.randn(1, 4 * world + 1, 2, 8), mode=1))
    rejects("moves no data", lambda: g.all_to_all_4d(torch.randn(1, 0, 2 * world, 8)))
    rejects("out has shape", lambda: g.all_to_all_4d(ok, out=torch.empty(1, 4 * world, 3, 8)))
    rejects("out has dtype", lambda: g.all_to_all_4d(ok, out=torch.empty(1, 4 * world, 2, 8).half()))
    rejects("contiguous CPU tensor",
            lambda: g.all_to_all_4d(ok, out=torch.empty(1, 2, 4 * world, 8).transpose(1, 2)))
    rejects("seq_splits has 0 entries", lambda: g.all_to_all_4d(ok, seq_splits=[], head_splits=[]))
    rejects("does not support torch.vmap", lambda: torch.vmap(lambda t: g.all_to_all_4d(t))(ok.unsqueeze(0)))
    rejects("transport must be", lambda: g.set_async_transport("dma"), exc=ValueError)
    # the transport setting is accepted on the CPU executor (where it has nothing to choose) and
    # the asynchronous call still delivers
    g.set_async_transport("copy_engine")
    assert torch.equal(g.all_to_all_4d_async(ok).wait(), g.all_to_all_4d(ok))
    g.set_async_transport("kernel")
    dist.barrier()
    # accepted: out= under no_grad with a grad-requiring input
    with torch.no_grad():
        g.all_to_all_4d(ok.clone().requires_grad_(), out=torch.empty(1, 4 * world, 2, 8))
    dist.barrier()
    g.destroy()
    rejects("has been destroyed", lambda: g.all_to_all_4d(ok))
    g.destroy()  # idempotent


def subgroups(rank, world):
    """tp x sp mesh: sp groups are the stride-2 subgroups, both run concurrently."""
    tp = 2
    sp = world // tp
    groups = [dist.new_group(list(range(t, world, tp))) for t in range(tp)]
    mine = groups[rank % tp]
    g = UlyssesGroup(mine, device="cpu")
    assert g.world_size == sp and g.rank == rank // tp
    x = torch.full((1, 3, 2 * sp, 8), float(rank))
    y = g.all_to_all_4d(x)
    # sequence block p of the output came from the p-th member of this sp group
    for p in range(sp):
        assert torch.all(y[:, 3 * p:3 * (p + 1)] == float(p * tp + rank % tp))
    g.destroy()


def fake_tensor(rank, world):
    from torch._subclasses.fake_tensor import FakeTensorMode

    g = UlyssesGroup(device="cpu")
    with FakeTensorMode():
        x = torch.empty(2, 5, 3 * world, 8)
        y = torch.ops.fast_ulysses_b200.all_to_all_4d(g._handle, x, 0, None, None)
        assert tuple(y.shape) == (2, 5 * world, 3, 8)
    g.destroy()


def fp8_exchange(rank, world):
    """Uneven heads [14, 13, 13]-style and +-10% sequence shards: the packed fp8 tensor goes through
    the same exchange, scales included, and matches the fp32 permutation up to fp8 rounding."""
    from fast_ulysses_b200.ops import fp8

    g = UlyssesGroup(device="cpu")
    heads = [5, 4, 4][:world]
    gen = torch.Generator().manual_seed(99)
    seq = [int(40 * (0.9 + 0.2 * torch.rand(1, generator=gen).item())) for _ in range(world)]
    torch.manual_seed(5 + rank)
    x = (torch.randn(1, seq[rank], sum(heads), 128) * 3).bfloat16()
    y = fp8.all_to_all_4d_fp8(g, x, mode=0, seq_splits=seq, head_splits=heads)
    want = reference_uneven(x.float(), 0, seq, heads, rank, world)
    assert y.shape == want.shape
    amax = want.abs().amax(-1, keepdim=True).clamp_min(1e-30)
    assert ((y.float() - want).abs() / amax).max() < 0.07
    # int8 payloads travel as bytes
    xi = torch.randint(-100, 100, (1, seq[rank], sum(heads), 128), dtype=torch.int8)
    yi = g.all_to_all_4d(xi, mode=0, seq_splits=seq, head_splits=heads)
    assert torch.equal(yi, reference_uneven(xi, 0, seq, heads, rank, world))
    g.destroy()
