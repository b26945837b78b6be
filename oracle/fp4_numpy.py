"""numpy restatement of the NVFP4 activation codec kyojin_mlx/fp4pack.py:21-63 (block 16, e4m3 scale) - TEST INFRASTRUCTURE, parity unpinned (the reference
implements it with MLX ops and compares it with a vendor function, neither of which is available here; the restatement follows the file line by line and
is cross-checked against an independent nearest-value formulation in tests/test_fp4pack_oracle.py)."""
from __future__ import annotations

import numpy as np

from .kq_numpy import e4m3_unsigned

LUT = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)


def e4m3_rn(v) -> np.ndarray:
    """float32 >= 0 -> e4m3fn byte, round to nearest even, saturating at 448 (mx.to_fp8)."""
    codes = np.arange(127, dtype=np.uint8)
    tab = e4m3_unsigned(codes).astype(np.float64)
    v = np.minimum(np.asarray(v, np.float64), 448.0)
    idx = np.clip(np.searchsorted(tab, v), 1, 126)
    lo, hi = tab[idx - 1], tab[idx]
    up = (v - lo > hi - v) | ((v - lo == hi - v) & (idx % 2 == 0))
    return np.where(up, idx, idx - 1).astype(np.uint8)


def _codes(v):
    mag = np.abs(v)
    code = sum((mag > t).astype(np.uint8) for t in (0.25, 1.25, 2.5, 5.0)) + sum((mag >= t).astype(np.uint8) for t in (0.75, 1.75, 3.5))
    return code | ((v < 0).astype(np.uint8) << 3)


def pack(x, block: int = 16, e4m3_scale: bool = True):
    """x [.., D] -> (codes uint8 [.., D/2], scale bytes uint8 [.., D/block]). (fp4pack.py:30-48, both branches: block 16 with an e4m3 scale, block 32 with the
    power-of-two scale 2^ceil(log2(amax / 6)) stored as exponent + 127; the ceiling is the mathematical one of the float32 quotient)"""
    x = np.asarray(x).astype(np.float32)
    shape = x.shape
    b = x.reshape(shape[:-1] + (-1, block))
    if e4m3_scale:
        amax = np.maximum(np.abs(b).max(-1, keepdims=True), np.float32(6.0 * 2.0 ** -9))
        s8 = e4m3_rn((amax / np.float32(6.0)).astype(np.float32))
        scale = e4m3_unsigned(s8)
    else:
        amax = np.maximum(np.abs(b).max(-1, keepdims=True), np.float32(6.0 * 2.0 ** -126))
        q = (amax / np.float32(6.0)).astype(np.float32)
        m, e = np.frexp(q.astype(np.float64))                               # q = m 2^e, 0.5 <= m < 1: ceil(log2 q) = e - 1 when m == 0.5, else e
        ce = np.where(m == 0.5, e - 1, e).astype(np.int32)
        s8 = (ce + 127).astype(np.uint8)
        scale = np.ldexp(np.float32(1.0), ce).astype(np.float32)
    v = np.clip((b / scale).astype(np.float32), -6.0, 6.0)
    code = _codes(v).reshape(shape[:-1] + (-1, 2))
    return (code[..., 0] | (code[..., 1] << 4)).astype(np.uint8).reshape(shape[:-1] + (shape[-1] // 2,)), s8.reshape(shape[:-1] + (shape[-1] // block,))


def unpack(codes, scales, block: int = 16, e4m3_scale: bool = True):
    """-> float32 [.., D] (fp4pack.py:51-63)."""
    codes = np.asarray(codes, np.uint8)
    d = codes.shape[-1] * 2
    c = np.stack([codes & 15, codes >> 4], -1).reshape(codes.shape[:-1] + (d,))
    val = np.where(c & 8, -LUT[c & 7], LUT[c & 7]).astype(np.float32)
    sc = e4m3_unsigned(np.asarray(scales, np.uint8)) if e4m3_scale else np.ldexp(np.float32(1.0), np.asarray(scales, np.int32) - 127).astype(np.float32)
    return (val.reshape(codes.shape[:-1] + (-1, block)) * sc[..., None]).reshape(codes.shape[:-1] + (d,)).astype(np.float32)
