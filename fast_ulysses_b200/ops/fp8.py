"""Block-scaled fp8 (e4m3, one fp32 scale per 128 values) payloads for the exchange.

``all_to_all_4d_fp8`` halves the bytes that cross NVLink: quantise (one scale per head of one
token), one ``all_to_all_4d`` on the packed ``(b, s, n, 144)`` uint8 tensor (the scale rides in
the same row as its payload, so a tile and its scale always arrive together), dequantise.
``quantize``/``dequantize`` fall back to plain PyTorch on CPU tensors (the plumbing tests).
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


def all_to_all_4d_fp8(group, x: torch.Tensor, *, mode: int = 0, seq_splits=None, head_splits=None) -> torch.Tensor:
    """``group.all_to_all_4d`` with the payload carried as block-scaled e4m3 (d must be 128)."""
    y = group.all_to_all_4d(quantize(x), mode=mode, seq_splits=seq_splits, head_splits=head_splits)
    return dequantize(y)
