"""Host-side weight container of the quantized linear (numpy only), mirroring kyojin_mlx/foreign_pack.py:39-86 `Pack`.

Pack(fmt, n, k, qs, meta, gscale, extra): n output rows, k inputs.
  fmt     qs                                                    meta
  q4_k    uint8 [n, k/256*144]  stored GGUF Q4_K rows            None
  q6_k    uint8 [n, k/256*210]  stored GGUF Q6_K rows            None
  q3_k    uint8 [n, k/256*110]  stored GGUF Q3_K rows            None
  q5_k    uint8 [n, k/256*176]  stored GGUF Q5_K rows            None
  q2_k    uint8 [n, k/256*84]   stored GGUF Q2_K rows            None
  iq4_xs  uint8 [n, k/256*136]  stored GGUF IQ4_XS rows          None
  q8_0    uint8 [n, k/32*34]    stored GGUF Q8_0 rows            None
  nvfp4   uint8 [n, k/2]  byte b = input 2b | input 2b+1 << 4    uint16 [n, k/32]: two e4m3 scale bytes (inputs 0-15, 16-31);
                                                                 gscale (float32) multiplies the row result
The reference's Pack keeps K-quant bits in arrays split for its Metal kernels (kyojin_mlx/foreign_gguf.py:725-789); here the K-quant
payload stays as stored and the device layout (T16, kyojin_mac_b200/layout.py) is produced when a DevPack is built. The NVFP4 form is
the reference's (and the safetensors files') own."""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from . import layout as L

FORMATS = L.FORMATS
GGUF_TO_FMT = {"Q4_K": "q4_k", "Q6_K": "q6_k", "Q3_K": "q3_k", "NVFP4": "nvfp4", "Q5_K": "q5_k", "Q8_0": "q8_0", "Q2_K": "q2_k", "IQ4_XS": "iq4_xs"}


@dataclass
class Pack:
    fmt: str
    n: int
    k: int
    qs: np.ndarray
    meta: np.ndarray | None = None
    gscale: float | np.ndarray = 1.0
    extra: dict = field(default_factory=dict)

    def __post_init__(self):
        if self.fmt not in FORMATS:
            raise ValueError(f"unknown foreign format {self.fmt} (this build serves {', '.join(FORMATS)})")
        if self.k <= 0 or self.k % L.KBLOCK:
            raise ValueError(f"{self.fmt}: k={self.k} is not a multiple of {L.KBLOCK}")
        if self.fmt == "nvfp4":
            if self.qs.shape != (self.n, self.k // 2) or self.qs.dtype != np.uint8:
                raise ValueError(f"nvfp4: qs {self.qs.shape} {self.qs.dtype} != uint8 [{self.n}, {self.k // 2}]")
            if self.meta is None or self.meta.shape != (self.n, self.k // 32) or self.meta.dtype != np.uint16:
                raise ValueError(f"nvfp4: meta must be uint16 [{self.n}, {self.k // 32}]")
        else:
            rb = L.raw_row_bytes(self.fmt, self.k)
            if self.qs.shape != (self.n, rb) or self.qs.dtype != np.uint8:
                raise ValueError(f"{self.fmt}: qs {self.qs.shape} {self.qs.dtype} != uint8 [{self.n}, {rb}] (stored GGUF rows)")

    @property
    def nbytes(self) -> int:
        return self.qs.nbytes + (0 if self.meta is None else self.meta.nbytes)


def to_pack(tname: str, raw, k: int) -> Pack:
    """Stored GGUF rows [n, row_bytes] of type `tname` -> Pack (role of kyojin_mlx/foreign_gguf.py:634 `to_pack`)."""
    if tname not in GGUF_TO_FMT:
        raise ValueError(f"GGUF type {tname} has no B200 kernel in this build (kernel types: {', '.join(GGUF_TO_FMT)})")
    fmt = GGUF_TO_FMT[tname]
    raw = np.ascontiguousarray(np.asarray(raw, np.uint8))
    n = raw.shape[0]
    if fmt == "nvfp4":
        codes, sc = L.nvfp4_raw_to_codes(raw, k)
        qs, meta = L.nvfp4_codes_to_pack(codes, sc)
        return Pack("nvfp4", n, k, qs, meta, 1.0)
    return Pack(fmt, n, k, raw)


def pack_nvfp4(weight_u8, scale_u8, gscale=1.0) -> Pack:
    """safetensors NVFP4 tensors (weight U8 [n, k/2], weight_scale e4m3 bytes [n, k/16], global scale) -> Pack
    (role of kyojin_mlx/foreign_pack.py:480-505 `pack_from_safetensors`)."""
    w = np.ascontiguousarray(np.asarray(weight_u8, np.uint8))
    n, k = w.shape[0], w.shape[1] * 2
    sc = np.ascontiguousarray(np.asarray(scale_u8, np.uint8)).reshape(n, k // 16)
    return Pack("nvfp4", n, k, w, sc.view("<u2").reshape(n, k // 32), gscale)


def to_t16(p: Pack) -> np.ndarray:
    """The pack's weights in the T16 device layout (host bytes)."""
    if p.fmt == "nvfp4":
        codes, sc = L.nvfp4_pack_to_codes(p.qs, p.meta)
        return L.nvfp4_codes_to_t16(codes, sc)
    return L.raw_to_t16(p.fmt, p.qs, p.n, p.k)


def concat_rows(packs) -> Pack:
    """Same-input members as one matrix (rows concatenated), as kyojin_mlx/foreign_pack.py:509-520 `concat_rows`."""
    p0 = packs[0]
    if any((p.fmt, p.k) != (p0.fmt, p0.k) for p in packs):
        raise ValueError("concat_rows: members differ in format or input width")
    if p0.fmt == "nvfp4" and any(float(np.asarray(p.gscale).reshape(-1)[0]) != float(np.asarray(p0.gscale).reshape(-1)[0]) for p in packs):
        raise ValueError("concat_rows: nvfp4 members with different global scales cannot share one matrix")
    qs = np.concatenate([p.qs for p in packs], 0)
    meta = None if p0.meta is None else np.concatenate([p.meta for p in packs], 0)
    return Pack(p0.fmt, sum(p.n for p in packs), p0.k, qs, meta, p0.gscale)
