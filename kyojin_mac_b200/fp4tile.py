"""Decode-friendly tile layout of NVFP4 expert stacks and its gathered GEMV: torch mirror of kyojin_mlx/fp4tile.py (`to_tile` :72-92, `from_tile` :111-134,
`tile_ref` :138-149, `gather` :298-302, `gather_glu` :305-309, `dequant` :317-321). The tile layout here is T16 (kyojin_mac_b200/layout.py): 16 rows x 256 inputs
per tile, codes bit-sliced for a shift-and-mask decode into fp16 operand pairs, scales beside them; same byte count as the stored arrays, exactly invertible."""
from __future__ import annotations

import numpy as np
import torch

from . import layout as L, ops


def tile_ok(n: int, k: int, ub: int = 2) -> bool:
    return n % 16 == 0 and k % 256 == 0


def to_tile(qs, meta, ub: int = 2, device="cuda") -> torch.Tensor:
    """Stored arrays qs uint32 [E, n, k/8] (8 e2m1 nibbles per word, element t = nibble t), meta uint16 [E, n, k/32] -> tile layout uint8 [E, tile bytes]."""
    qs, meta = np.asarray(qs.cpu() if isinstance(qs, torch.Tensor) else qs), np.asarray(meta.cpu() if isinstance(meta, torch.Tensor) else meta)
    E, n, k8 = qs.shape
    out = []
    for e in range(E):
        q8 = np.ascontiguousarray(qs[e].astype("<u4")).view(np.uint8).reshape(n, k8 * 4)       # byte b = element 2b | element 2b+1 << 4
        codes, sc = L.nvfp4_pack_to_codes(q8, np.ascontiguousarray(meta[e]).astype("<u2"))
        out.append(L.nvfp4_codes_to_t16(codes, sc))
    return torch.from_numpy(np.stack(out)).to(device)


def from_tile(tl: torch.Tensor, n: int, k: int, ub: int = 2):
    """Tile layout -> (qs uint32 [E, n, k/8], meta uint16 [E, n, k/32]) numpy arrays in the stored layout."""
    t = tl.cpu().numpy()
    qs, meta = [], []
    for e in range(t.shape[0]):
        codes, sc = L.t16_to_nvfp4_codes(t[e], n, k)
        q8, m = L.nvfp4_codes_to_pack(codes, sc)
        qs.append(np.ascontiguousarray(q8).view("<u4").reshape(n, k // 8))
        meta.append(m)
    return np.stack(qs), np.stack(meta)


def tile_ref(qs, meta, gs) -> np.ndarray:
    """float64 [E, n, k] dequant of the STORED arrays (the reference both layouts are compared with; kyojin_mlx/fp4tile.py:138-149)."""
    qs, meta = np.asarray(qs), np.asarray(meta)
    E, n, k8 = qs.shape
    nib = ((qs[..., None] >> (4 * np.arange(8, dtype=np.uint32))) & 15).reshape(E, n, k8 * 8)
    lut = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], np.float64)
    v = lut[nib & 7] * np.where(nib & 8, -1.0, 1.0)
    sb = np.ascontiguousarray(meta).view(np.uint8).reshape(E, n, k8 * 8 // 16).astype(np.int64) & 127
    ex, m = sb >> 3, sb & 7
    sc = np.where(ex == 0, m * 2.0 ** -9, 2.0 ** (ex - 7.0) * (1 + m / 8.0))
    sc = np.where(sb == 127, 0.0, sc)
    return v * np.repeat(sc, 16, axis=-1) * np.asarray(gs, np.float64).reshape(E, 1, 1)


def gather(x, xrows, eids, tl, gs, n: int, k: int, ub: int = 2, nsg: int = 4, mode: str = "", pf: int = 1) -> torch.Tensor:
    """y fp16 [S, n]: slot s = expert eids[s] applied to row xrows[s] of x (fp16 [T, k])."""
    E = tl.shape[0]
    return ops.gemv_group("nvfp4", tl.reshape(-1), n, k, E, x, eids, xrows=xrows, gs=gs)


def gather_glu(x, xrows, eids, tl_g, tl_u, gs_g, gs_u, n: int, k: int, limit=None, ub: int = 2, nsg: int = 8, pf: int = 1, act=None) -> torch.Tensor:
    """h fp16 [S, n] = glu(gate(x), up(x)) for each slot."""
    if act is not None:
        raise NotImplementedError("only the silu-gated activation is built")
    return ops.silu_mul(gather(x, xrows, eids, tl_g, gs_g, n, k), gather(x, xrows, eids, tl_u, gs_u, n, k), limit)


def dequant(tl, gs, E: int, n: int, k: int, ub: int = 2) -> torch.Tensor:
    """float16 [E, n, k] of a tile-layout stack."""
    out = torch.empty((E, n, k), dtype=torch.float16, device=tl.device)
    flat = tl.reshape(-1)
    for e in range(E):
        out[e] = ops.dequant("nvfp4", flat, E * n, k, torch.float16, float(gs[e]), e * n, n)
    return out
