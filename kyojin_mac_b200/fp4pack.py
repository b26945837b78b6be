"""NVFP4 / MXFP4-style activation codec on the device: torch mirror of kyojin_mlx/fp4pack.py (`pack` :30-48, `unpack` :51-63) for the block-16, e4m3-scale
form (the NVFP4 rule). The block-32 power-of-two (e8m0) form of the reference's index keys is not part of the quantized-linear path and is not built."""
from __future__ import annotations

import torch

from . import ops


def pack(x: torch.Tensor, block: int = 16, e4m3_scale: bool = True):
    """x [.., D] fp16 / bf16 -> (codes uint8 [.., D // 2], scales uint8 [.., D // block]); same rounding as the reference (amax / 6 -> e4m3, clip to +-6,
    round to nearest even onto e2m1, sign bit 3, two codes per byte low first)."""
    if block != 16 or not e4m3_scale:
        raise NotImplementedError("only block = 16 with e4m3 scales (NVFP4) is built")
    shape = x.shape
    if shape[-1] % 16:
        raise ValueError("last dimension must be a multiple of 16")
    x2 = x.reshape(-1, shape[-1])
    if x2.dtype not in (torch.float16, torch.bfloat16):
        x2 = x2.to(torch.float16)
    codes, sp, _ = ops.nvfp4_quant_rows(x2.contiguous(), swizzled=False, plain=True)
    return codes.reshape(*shape[:-1], shape[-1] // 2), sp.reshape(*shape[:-1], shape[-1] // 16)


def unpack(codes: torch.Tensor, scales: torch.Tensor, block: int = 16, e4m3_scale: bool = True, dtype=torch.float16):
    if block != 16 or not e4m3_scale:
        raise NotImplementedError("only block = 16 with e4m3 scales (NVFP4) is built")
    lead = codes.shape[:-1]
    d = codes.shape[-1] * 2
    out = ops.nvfp4_unpack_rows(codes.reshape(-1, d // 2).contiguous(), scales.reshape(-1, d // 16).contiguous(), dtype)
    return out.reshape(*lead, d)
