"""Seeded synthetic weights with the shapes and value distributions of the benchmark configurations: random payload bytes
with sane fp16 scale fields, the same rule as the reference's test generator (kyojin_mlx/foreign_synth.py:32-44
`random_blocks`: "random bit patterns with sane fp16 scales"). They stand in for real model files, which are not available.

numpy versions produce stored GGUF rows (for parity tests against the oracle); torch versions write T16 tiles directly on
the device for the full-size benchmark (a T16 tile of random bytes IS a repacked random block: the repack is a bit permutation;
only the fp16 scale fields are placed explicitly)."""
from __future__ import annotations

import numpy as np

from .layout import KBLOCK, RAW_BLOCK, TILE_BYTES, padded_rows

# byte offsets of the fp16 scale fields inside a stored block / inside a T16 tile (per row r)
_RAW_F16 = {"q4_k": (0, 2), "q6_k": (208,), "q3_k": (108,), "q5_k": (0, 2), "q8_0": (0,), "q2_k": (80, 82), "iq4_xs": (0,)}
_T16_F16 = {"q4_k": (2048, 16, (0, 2)), "q6_k": (3328, 2, (0,)), "q3_k": (1728, 2, (0,)), "q5_k": (2560, 16, (0, 2)),
            "q8_0": (4096, 16, (0, 2, 4, 6, 8, 10, 12, 14)), "q2_k": (1280, 4, (0, 2)), "iq4_xs": (2048, 8, (0,))}     # region offset, row stride, field offsets


def raw_blocks(fmt: str, n: int, k: int, rng: np.random.Generator, d_sigma: float = 1e-3) -> np.ndarray:
    """uint8 [n, row_bytes] of stored blocks: uniform random bytes; d (and dmin) = fp16(|N(0, d_sigma)|); Q6_K int8 scales are any
    byte (the configuration's U[-32, 31] is set by `q6k_scale_range`); NVFP4 scale bytes: e4m3 nearest to 2^U[-8, 0]."""
    be, bb = RAW_BLOCK[fmt]
    b = rng.integers(0, 256, (n, k // be, bb), dtype=np.uint8)
    if fmt == "nvfp4":
        b[..., 0:4] = nvfp4_scale_bytes(rng, (n, k // be, 4))
    else:
        for off in _RAW_F16[fmt]:
            b[..., off:off + 2] = np.abs(rng.normal(0.0, d_sigma, (n, k // be))).astype("<f2").view(np.uint8).reshape(n, k // be, 2)
        if fmt == "q6_k":
            b[..., 192:208] = rng.integers(-32, 32, (n, k // be, 16)).astype(np.int8).view(np.uint8)
    return np.ascontiguousarray(b.reshape(n, -1))


def nvfp4_scale_bytes(rng: np.random.Generator, shape) -> np.ndarray:
    """e4m3 byte nearest (ties to even) to 2^u, u ~ U[-8, 0]: exercises mantissa bits and the subnormal range below 2^-6."""
    v = np.exp2(rng.uniform(-8.0, 0.0, shape)).astype(np.float32)
    return e4m3_round(v)


def e4m3_round(v: np.ndarray) -> np.ndarray:
    """float32 >= 0 -> nearest e4m3fn byte (round to nearest even, saturating at 448), via the table of the 127 finite codes."""
    codes = np.arange(127, dtype=np.uint8)
    e, m = (codes >> 3).astype(np.int32), (codes & 7).astype(np.float64)
    tab = np.where(e == 0, np.ldexp(m, -9), np.ldexp(1.0 + m / 8.0, e - 7))
    v = np.asarray(v, np.float64)
    idx = np.clip(np.searchsorted(tab, v), 1, 126)
    lo, hi = tab[idx - 1], tab[idx]
    pick_hi = (v - lo > hi - v) | ((v - lo == hi - v) & (idx % 2 == 0))
    return np.where(pick_hi, idx, idx - 1).astype(np.uint8)


def activations(m: int, k: int, rng: np.random.Generator) -> np.ndarray:
    return rng.standard_normal((m, k)).astype(np.float16)


def t16_random_device(fmt: str, n: int, k: int, seed: int, device="cuda", d_sigma: float = 1e-3):
    """T16 tiles of a random matrix, generated on the device (torch): uniform random bytes, then the scale fields overwritten."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    ntile = padded_rows(n) // 16 * (k // KBLOCK)
    tb = TILE_BYTES[fmt]
    # int32 draws viewed as bytes: torch has no uint8 generator on full range that is faster
    t = torch.randint(-2 ** 31, 2 ** 31 - 1, (ntile, tb // 4), dtype=torch.int32, device=device, generator=g).view(torch.uint8).reshape(ntile, tb)
    if fmt == "nvfp4":
        u = torch.rand((ntile, 256), device=device, generator=g) * -8.0
        t[:, 2048:2304] = _e4m3_round_torch(torch.exp2(u))
        return t.reshape(-1)
    off, stride, fields = _T16_F16[fmt]
    for f in fields:
        d = (torch.randn((ntile, 16), device=device, generator=g) * d_sigma).abs().to(torch.float16).view(torch.uint8).reshape(ntile, 16, 2)
        idx = off + torch.arange(16, device=device) * stride + f
        t[:, idx] = d[:, :, 0]
        t[:, idx + 1] = d[:, :, 1]
    if fmt == "q6_k":
        sc = torch.randint(-32, 32, (ntile, 256), dtype=torch.int8, device=device, generator=g).view(torch.uint8)
        t[:, 3072:3328] = sc
    return t.reshape(-1)


def _e4m3_round_torch(v):
    import torch
    return v.to(torch.float8_e4m3fn).view(torch.uint8)
