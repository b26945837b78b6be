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


def pack(x):
    """x [.., D] -> (codes uint8 [.., D/2], scale bytes uint8 [.., D/16]). (fp4pack.py:30-48)"""
    x = np.asarray(x).astype(np.float32)
    shape = x.shape
    b = x.reshape(shape[:-1] + (-1, 16))
    amax = np.maximum(np.abs(b).max(-1, keepdims=True), np.float32(6.0 * 2.0 ** -9))
    s8 = e4m3_rn((amax / np.float32(6.0)).astype(np.float32))
    scale = e4m3_unsigned(s8)
    v = np.clip((b / scale).astype(np.float32), -6.0, 6.0)
    mag = np.abs(v)
    code = sum((mag > t).astype(np.uint8) for t in (0.25, 1.25, 2.5, 5.0)) + sum((mag >= t).astype(np.uint8) for t in (0.75, 1.75, 3.5))
    code = (code | ((v < 0).astype(np.uint8) << 3)).reshape(shape[:-1] + (-1, 2))
    return (code[..., 0] | (code[..., 1] << 4)).astype(np.uint8).reshape(shape[:-1] + (shape[-1] // 2,)), s8.reshape(shape[:-1] + (shape[-1] // 16,))


def unpack(codes, scales):
    """-> float32 [.., D] (fp4pack.py:51-63)."""
    codes = np.asarray(codes, np.uint8)
    d = codes.shape[-1] * 2
    c = np.stack([codes & 15, codes >> 4], -1).reshape(codes.shape[:-1] + (d,))
    val = np.where(c & 8, -LUT[c & 7], LUT[c & 7]).astype(np.float32)
    sc = e4m3_unsigned(np.asarray(scales, np.uint8))
    return (val.reshape(codes.shape[:-1] + (-1, 16)) * sc[..., None]).reshape(codes.shape[:-1] + (d,)).astype(np.float32)
