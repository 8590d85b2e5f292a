"""Block-scaled fp8 (e4m3, one fp32 scale per 128 values) payloads for the exchange.

``all_to_all_4d_fp8`` sends 0.56 of the bf16 bytes over NVLink. On a CUDA group it is ONE kernel
(csrc/kernels/quant.cu: fu_a2a4d_fp8): every (token, head) row is quantised in registers on its way
into the owning peer's window (the scale rides in the same 144-byte row as its payload, so a row
and its scale always arrive together) and the window is expanded into the bf16 result after the
closing handshake; the quantisation costs no pass of its own over HBM. On the CPU/gloo backend, and
with ``fused=False``, it is the composition quantise -> ``all_to_all_4d`` of the packed uint8 tensor
-> dequantise. ``quantize``/``dequantize`` fall back to plain PyTorch on CPU tensors.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _ckernels as ck

BLOCK, PACKED = 128, 144


def quantize(x: torch.Tensor) -> torch.Tensor:
    """(..., 128) bf16 -> (..., 144) uint8."""
    assert x.shape[-1] == BLOCK and x.dtype == torch.bfloat16
    x = x.contiguous()
    out = torch.empty(*x.shape[:-1], PACKED, dtype=torch.uint8, device=x.device)
    blocks = x.numel() // BLOCK
    if x.is_cuda:
        lib = ck.lib()
        lib.fu_quant_e4m3_block128.restype = C.c_int
        lib.fu_quant_e4m3_block128.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
        ck.check(lib.fu_quant_e4m3_block128(x.data_ptr(), out.data_ptr(), blocks, ck.stream_ptr()))
        return out
    xf = x.float().reshape(-1, BLOCK)
    amax = xf.abs().amax(dim=1, keepdim=True)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    q = (xf / scale).clamp(-448, 448).to(torch.float8_e4m3fn)
    flat = out.view(-1, PACKED)
    flat[:, :BLOCK] = q.view(torch.uint8)
    flat[:, BLOCK:] = 0
    flat[:, BLOCK:BLOCK + 4] = scale.to(torch.float32).view(torch.uint8).reshape(-1, 4)
    return out


def dequantize(packed: torch.Tensor) -> torch.Tensor:
    """(..., 144) uint8 -> (..., 128) bf16."""
    assert packed.shape[-1] == PACKED and packed.dtype == torch.uint8
    packed = packed.contiguous()
    out = torch.empty(*packed.shape[:-1], BLOCK, dtype=torch.bfloat16, device=packed.device)
    blocks = packed.numel() // PACKED
    if packed.is_cuda:
        lib = ck.lib()
        lib.fu_dequant_e4m3_block128.restype = C.c_int
        lib.fu_dequant_e4m3_block128.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
        ck.check(lib.fu_dequant_e4m3_block128(packed.data_ptr(), out.data_ptr(), blocks, ck.stream_ptr()))
        return out
    flat = packed.view(-1, PACKED)
    scale = flat[:, BLOCK:BLOCK + 4].contiguous().view(torch.float32)
    q = flat[:, :BLOCK].contiguous().view(torch.float8_e4m3fn).float()
    out.view(-1, BLOCK).copy_((q * scale).to(torch.bfloat16))
    return out


def all_to_all_4d_fp8(group, x: torch.Tensor, *, mode: int = 0, seq_splits=None, head_splits=None,
                      fused: bool = True) -> torch.Tensor:
    """``group.all_to_all_4d`` with the payload carried as block-scaled e4m3 (d must be 128, bf16).
    Collective; the first call of a larger size allocates a symmetric window (every rank together)."""
    if not (fused and x.is_cuda):
        y = group.all_to_all_4d(quantize(x), mode=mode, seq_splits=seq_splits, head_splits=head_splits)
        return dequantize(y)
    return _fused_exchange(group, x, mode, seq_splits, head_splits)


def _fused_exchange(group, x, mode, seq_splits, head_splits):
    assert x.dim() == 4 and x.shape[-1] == BLOCK and x.dtype == torch.bfloat16, (x.shape, x.dtype)
    if (seq_splits is None) != (head_splits is None):
        raise RuntimeError("pass both seq_splits and head_splits, or neither")
    world, rank = group.world_size, group.rank
    b, s, n, _ = x.shape
    if seq_splits is None:  # even shards, as in all_to_all_4d
        if mode == 0:
            if n % world:
                raise RuntimeError(f"mode 0 scatters the head axis, so n_global ({n}) must divide world_size ({world})")
            seq_splits, head_splits = [s] * world, [n // world] * world
        else:
            if s % world:
                raise RuntimeError(f"mode 1 scatters the sequence axis, so s_global ({s}) must divide world_size ({world})")
            seq_splits, head_splits = [s // world] * world, [n] * world
    x = x.contiguous()
    out_shape, window_numel, sends, _, _ = torch.ops.fast_ulysses_b200.a2a_plan_debug(b, BLOCK, rank, world, list(seq_splits),
                                                                list(head_splits), mode, 2)
    win_bytes = window_numel // BLOCK * PACKED  # packed bytes of the largest result of any rank
    cache = group._fp8_window  # one symmetric window per group, grown collectively, dropped by destroy()
    if cache.get("bytes", 0) < win_bytes:  # collective: every rank computes the same size
        buf = group._handle.symm_alloc(win_bytes)
        ptrs = group._handle.symm_ptrs(buf)
        cache.update(bytes=win_bytes, buf=buf, base=list(ptrs[:world]), ctrl=list(ptrs[world:]))
    out = torch.empty(tuple(out_shape), dtype=torch.bfloat16, device=x.device)
    a = ck.FuA2AFp8Args()
    a.src, a.out = x.data_ptr(), out.data_ptr()
    for p in range(world):
        a.peer_win[p], a.peer_ctrl[p] = cache["base"][p], cache["ctrl"][p]
    a.win_bytes, a.src_bytes, a.out_rows = cache["bytes"], x.numel() * 2, out.numel() // BLOCK
    a.rank, a.world = rank, world
    rows = sends.tolist()
    # start with the next rank up, as the bf16 exchange does, so every rank's ingress has one sender at a time
    rows.sort(key=lambda r: (int(r[0]) - rank - 1) % world)
    a.n_routes = len(rows)
    for i, row in enumerate(rows):
        a.routes[i] = ck.route_from_row(row)
    a.timeout_ms = int(getattr(group, "timeout_ms", 10000) or 10000)
    ck.check(ck.lib().fu_a2a4d_fp8(C.byref(a), ck.stream_ptr()))
    return out
