"""NVFP4 / MXFP4-style activation codec on the device: torch mirror of kyojin_mlx/fp4pack.py (`pack` :30-48, `unpack` :51-63), both forms: block 16 with an
e4m3 scale (the NVFP4 rule, also the quantiser of the W4A4 prefill GEMM) and block 32 with a power-of-two scale stored as an exponent byte."""
from __future__ import annotations

import torch

from . import _lib, ops


def _form(block: int, e4m3_scale: bool) -> bool:
    if (block, bool(e4m3_scale)) == (16, True):
        return True
    if (block, bool(e4m3_scale)) == (32, False):
        return False
    raise ValueError("the codec has two forms: block = 16 with e4m3 scales, block = 32 with power-of-two scales")


def pack(x: torch.Tensor, block: int = 16, e4m3_scale: bool = True):
    """x [.., D] fp16 / bf16 -> (codes uint8 [.., D // 2], scales uint8 [.., D // block]); same rounding as the reference (block 16: amax / 6 -> e4m3;
    block 32: 2^ceil(log2(amax / 6)) as exponent + 127; clip to +-6, round to nearest even onto e2m1, sign bit 3, two codes per byte low first)."""
    nv = _form(block, e4m3_scale)
    shape = x.shape
    if shape[-1] % block:
        raise ValueError(f"last dimension must be a multiple of {block}")
    x2 = x.reshape(-1, shape[-1])
    if x2.dtype not in (torch.float16, torch.bfloat16):
        x2 = x2.to(torch.float16)
    x2 = x2.contiguous()
    if nv:
        codes, sp, _ = ops.nvfp4_quant_rows(x2, swizzled=False, plain=True)
    else:
        ops._need_cuda(x2)
        rows, k = x2.shape
        codes = torch.empty((rows, k // 2), dtype=torch.uint8, device=x2.device)
        sp = torch.empty((rows, k // 32), dtype=torch.uint8, device=x2.device)
        _lib.check(_lib.lib().kyb_fp4_quant_block32(x2.data_ptr(), ops._DT[x2.dtype], x2.stride(0), rows, k, codes.data_ptr(), sp.data_ptr(), ops._stream()))
    return codes.reshape(*shape[:-1], shape[-1] // 2), sp.reshape(*shape[:-1], shape[-1] // block)


def unpack(codes: torch.Tensor, scales: torch.Tensor, block: int = 16, e4m3_scale: bool = True, dtype=torch.float16):
    nv = _form(block, e4m3_scale)
    lead = codes.shape[:-1]
    d = codes.shape[-1] * 2
    c2, s2 = codes.reshape(-1, d // 2).contiguous(), scales.reshape(-1, d // block).contiguous()
    if nv:
        out = ops.nvfp4_unpack_rows(c2, s2, dtype)
    else:
        ops._need_cuda(c2, s2)
        out = torch.empty((c2.shape[0], d), dtype=dtype, device=c2.device)
        _lib.check(_lib.lib().kyb_fp4_unpack_block32(c2.data_ptr(), s2.data_ptr(), c2.shape[0], d, ops._DT[dtype], out.data_ptr(), d, ops._stream()))
    return out.reshape(*lead, d)
