"""T16: the HBM layout the sm_100a kernels stream (numpy side: load-time repack and its inverse).

A matrix [n, k] (k % 256 == 0) is cut into tiles of 16 output rows x 256 inputs. Tile (rt, kb) sits at byte
((rt * k/256) + kb) * TILE_BYTES[fmt]: all the bytes one warp needs for one k-block of its 16 rows are contiguous (one
bulk copy) and the k-blocks of a row tile follow each other, so a warp reads one linear stream. Inside a tile the quant
bits are ordered so that lane L = 4 g + t of a warp finds, with 128-bit shared-memory loads, exactly the register
operands of `mma.sync.m16n8k16` for rows g and g + 8: MMA number s of a tile covers inputs 16 s .. 16 s + 15, and lane t
owns inputs 16 s + 4 t + b, b = 0..3 ("byte quad").  The repack is a permutation of the stored bits: same byte count as
the GGUF blocks (144 / 210 / 110 bytes per 256 weights, NVFP4 144), nothing re-quantised, exactly invertible.
n is padded with zero blocks to a multiple of 16 (a zero block decodes to zeros in every format).

It plays the role of the reference's lossless load-time repack (kyojin_mlx/foreign_gguf.py:634-789 `to_pack`, and the
decode-friendly tile layout of kyojin_mlx/fp4tile.py:72-92), re-designed for 16-row tensor-core fragments and bulk copies.

Tile contents (offsets in bytes; "word(P, L, i)" = 32-bit word i of the 16-byte unit of lane L in plane slice P):
  q4_k  [0,2048)    word(G, L, 2c+h) = stored quant word 8G + 4c + t of row g + 8h: byte b = input 64G+16c+4t+b (low nibble, sub-block 2G)
                    and input 64G+32+16c+4t+b (high nibble, sub-block 2G+1)
        [2048,2304) row r: the first 16 stored bytes of its block (d, dmin, 12 bytes of 6-bit scales/mins)
  q6_k  [0,2048)    word(P, L, 2p+h): byte b = low 4 bits of input 16 s0+4t+b | low 4 bits of input 16 s1+4t+b << 4, s0 = 4P+2p, s1 = s0+1
        [2048,3072) word(P2, L, 2a+h): byte b, bits 2i..2i+1 = high 2 bits of input 16 (8 P2 + 4a + i) + 4t + b
        [3072,3328) row r: 16 int8 scales     [3328,3360) row r: fp16 d
  q3_k  [0,1024)    word(P2, L, 2a+h): byte b, bits 2i..2i+1 = low 2 bits of input 16 (8 P2 + 4a + i) + 4t + b
        [1024,1536) word(0, L, 2a+h): byte b, bit i = high bit of input 16 (8a + i) + 4t + b
        [1536,1728) row r: the 12 stored scale bytes     [1728,1760) row r: fp16 d
  nvfp4 [0,2048)    word(P, L, 2p+h) holds 8 e2m1 codes bit-sliced for a shift-and-mask decode straight into fp16 pairs: the low/high 16 bits
                    carry the first/second input of the pairs (4t, 4t+2) [v0], (4t+1, 4t+3) [v1] of MMA s0 = 4P+2p and the same of s1 [v2, v3];
                    magnitude bits of v0..v3 at [11:9], [8:6], [5:3], [2:0], sign bits at 15, 12, 13, 14
        [2048,2304) row r: 16 e4m3 scale bytes (one per 16 inputs)
  q5_k  [0,2048)    the low 4 bits of the 5-bit codes as the q6_k nibble plane   [2048,2560) the fifth bits as the q3_k 1-bit plane
        [2560,2816) row r: the first 16 stored bytes of its block (d, dmin, 12 bytes of 6-bit scales/mins)
  q8_0  [0,4096)    word(P, L, 2p+h): byte b = the int8 of input 16 (2P + p) + 4t + b       [4096,4352) row r: the eight fp16 d of its 32-input blocks
  iq4_xs [0,2048)   the 4-bit grid indices as the q6_k nibble plane     [2048,2176) row r: the first 8 stored bytes of its block (d, scales_h, scales_l)
  q2_k  [0,1024)    the 2-bit codes as the q3_k 2-bit plane     [1024,1280) row r: the 16 stored scale | min << 4 bytes     [1280,1344) row r: fp16 d, fp16 dmin
"""
from __future__ import annotations

import numpy as np

FORMATS = ("q4_k", "q6_k", "q3_k", "nvfp4", "q5_k", "q8_0", "q2_k", "iq4_xs")
FMT_ID = {"q4_k": 0, "q6_k": 1, "q3_k": 2, "nvfp4": 3, "q5_k": 4, "q8_0": 5, "q2_k": 6, "iq4_xs": 7}
TILE_BYTES = {"q4_k": 2304, "q6_k": 3360, "q3_k": 1760, "nvfp4": 2304, "q5_k": 2816, "q8_0": 4352, "q2_k": 1344, "iq4_xs": 2176}
RAW_BLOCK = {"q4_k": (256, 144), "q6_k": (256, 210), "q3_k": (256, 110), "nvfp4": (64, 36), "q5_k": (256, 176), "q8_0": (32, 34), "q2_k": (256, 84), "iq4_xs": (256, 136)}     # GGUF block elements / bytes
GGUF_NAME = {"q4_k": "Q4_K", "q6_k": "Q6_K", "q3_k": "Q3_K", "nvfp4": "NVFP4", "q5_k": "Q5_K", "q8_0": "Q8_0", "q2_k": "Q2_K", "iq4_xs": "IQ4_XS"}
PREFILL_FUSED = FORMATS                                 # formats the prefill GEMM decodes inside the kernel (all of them; the staged form stays an option)
ROWS = 16
KBLOCK = 256


def padded_rows(n: int) -> int:
    return (n + ROWS - 1) // ROWS * ROWS


def t16_nbytes(fmt: str, n: int, k: int) -> int:
    _check(fmt, k)
    return padded_rows(n) // ROWS * (k // KBLOCK) * TILE_BYTES[fmt]


def raw_row_bytes(fmt: str, k: int) -> int:
    be, bb = RAW_BLOCK[fmt]
    return k // be * bb


def _check(fmt, k):
    if fmt not in TILE_BYTES:
        raise ValueError(f"unknown format {fmt!r} (supported: {', '.join(FORMATS)})")
    if k <= 0 or k % KBLOCK:
        raise ValueError(f"{fmt}: k={k} must be a positive multiple of {KBLOCK}")


def _pad_rows(a, n):
    npad = padded_rows(n)
    if npad == n:
        return a
    z = np.zeros((npad - n,) + a.shape[1:], a.dtype)
    return np.concatenate([a, z], 0)


def _by_tile(a):
    """[npad, nb, ...] -> [nrt, nb, h2, g8, ...] (row r = 8 h + g of tile rt)."""
    npad, nb = a.shape[:2]
    a = a.reshape((npad // ROWS, 2, 8, nb) + a.shape[2:])
    return np.moveaxis(a, 3, 1)


def _from_tile(a):
    """inverse of _by_tile: [nrt, nb, h2, g8, ...] -> [npad, nb, ...]."""
    a = np.moveaxis(a, 1, 3)
    return a.reshape((a.shape[0] * ROWS, a.shape[3]) + a.shape[4:])


# ------------------------------------------------------------------------------------------------ planes
def _nibble_plane(lo4):
    """lo4 uint8 [nrt, nb, h, g, 256] (4-bit fields, natural input order) -> bytes [nrt, nb, 2048]."""
    a = lo4.reshape(lo4.shape[:4] + (4, 2, 2, 4, 4))                      # P, p, u, t, b   (s = 4P + 2p + u)
    byte = a[..., 0, :, :] | (a[..., 1, :, :] << 4)                         # [nrt, nb, h, g, P, p, t, b]
    out = byte.transpose(0, 1, 4, 3, 6, 5, 2, 7)                             # P, g, t, p, h, b
    return np.ascontiguousarray(out).reshape(out.shape[:2] + (2048,))


def _nibble_plane_inv(plane):
    a = plane.reshape(plane.shape[:2] + (4, 8, 4, 2, 2, 4))                # P, g, t, p, h, b
    a = a.transpose(0, 1, 6, 3, 2, 5, 4, 7)                                 # h, g, P, p, t, b
    lo4 = np.stack([a & 15, a >> 4], 6)                                     # h, g, P, p, u, t, b
    return np.ascontiguousarray(lo4).reshape(lo4.shape[:4] + (256,))


def _twobit_plane(f2):
    """f2 uint8 [nrt, nb, h, g, 256] (2-bit fields) -> bytes [nrt, nb, 1024]."""
    a = f2.reshape(f2.shape[:4] + (2, 2, 4, 4, 4))                         # P2, a, i, t, b   (s = 8 P2 + 4a + i)
    byte = a[..., 0, :, :] | (a[..., 1, :, :] << 2) | (a[..., 2, :, :] << 4) | (a[..., 3, :, :] << 6)   # h, g, P2, a, t, b
    out = byte.transpose(0, 1, 4, 3, 6, 5, 2, 7)                             # P2, g, t, a, h, b
    return np.ascontiguousarray(out).reshape(out.shape[:2] + (1024,))


def _twobit_plane_inv(plane):
    a = plane.reshape(plane.shape[:2] + (2, 8, 4, 2, 2, 4))                # P2, g, t, a, h, b
    a = a.transpose(0, 1, 6, 3, 2, 5, 4, 7)                                 # h, g, P2, a, t, b
    f = np.stack([(a >> (2 * i)) & 3 for i in range(4)], 6)                 # h, g, P2, a, i, t, b
    return np.ascontiguousarray(f).reshape(f.shape[:4] + (256,))


def _onebit_plane(f1):
    """f1 uint8 [nrt, nb, h, g, 256] (1-bit fields) -> bytes [nrt, nb, 512]."""
    a = f1.reshape(f1.shape[:4] + (2, 8, 4, 4))                            # a, i, t, b   (s = 8a + i)
    byte = np.zeros(a.shape[:5] + (4, 4), np.uint8)
    for i in range(8):
        byte |= a[..., i, :, :] << i                                        # h, g, a, t, b
    out = byte.transpose(0, 1, 3, 5, 4, 2, 6)                                # g, t, a, h, b
    return np.ascontiguousarray(out).reshape(out.shape[:2] + (512,))


def _onebit_plane_inv(plane):
    a = plane.reshape(plane.shape[:2] + (8, 4, 2, 2, 4))                   # g, t, a, h, b
    a = a.transpose(0, 1, 5, 2, 4, 3, 6)                                    # h, g, a, t, b
    f = np.stack([(a >> i) & 1 for i in range(8)], 5)                       # h, g, a, i, t, b
    return np.ascontiguousarray(f).reshape(f.shape[:4] + (256,))


_FP4_MAG_AT = (9, 6, 3, 0)
_FP4_SIGN_AT = (15, 12, 13, 14)


def _fp4_plane(codes):
    """codes uint8 [nrt, nb, h, g, 256] (e2m1 nibbles, natural order) -> bytes [nrt, nb, 2048] of bit-sliced words."""
    # input 16 s + 4t + b with s = 4P + 2p + u and b = 2j + e: pair v = 2u + e holds inputs b = e (low half, j = 0) and b = e + 2 (high half, j = 1)
    a = codes.reshape(codes.shape[:4] + (4, 2, 2, 4, 2, 2)).astype(np.uint32)   # P, p, u, t, j, e
    w = np.zeros(codes.shape[:4] + (4, 2, 4), np.uint32)                      # h, g, P, p, t
    for u in range(2):
        for e in range(2):
            v = 2 * u + e
            for j in range(2):
                c = a[..., u, :, j, e]                                         # [.., P, p, t]
                w |= ((c & 7) << (_FP4_MAG_AT[v] + 16 * j)) | ((c >> 3) << (_FP4_SIGN_AT[v] + 16 * j))
    out = w.transpose(0, 1, 4, 3, 6, 5, 2)                                      # P, g, t, p, h
    return np.ascontiguousarray(out.astype("<u4")).view(np.uint8).reshape(out.shape[:2] + (2048,))


def _fp4_plane_inv(plane):
    w = np.ascontiguousarray(plane).view("<u4").reshape(plane.shape[:2] + (4, 8, 4, 2, 2)).astype(np.uint32)   # P, g, t, p, h
    w = w.transpose(0, 1, 6, 3, 2, 5, 4)                                        # h, g, P, p, t
    codes = np.zeros(w.shape[:6] + (2, 4, 2, 2), np.uint8)                       # h, g, P, p, u, t, j, e
    for u in range(2):
        for e in range(2):
            v = 2 * u + e
            for j in range(2):
                mag = (w >> (_FP4_MAG_AT[v] + 16 * j)) & 7
                sg = (w >> (_FP4_SIGN_AT[v] + 16 * j)) & 1
                codes[..., u, :, j, e] = (mag | (sg << 3)).astype(np.uint8)
    return np.ascontiguousarray(codes).reshape(codes.shape[:4] + (256,))


# ------------------------------------------------------------------------------------------------ per format
def _q6k_codes(B):
    """[.., 210] -> 6-bit codes [.., 256] in natural input order (kyojin_mlx/foreign_gguf.py:481-488 element order)."""
    ql = B[..., 0:128].reshape(B.shape[:-1] + (2, 2, 32))                  # half128, which 32-byte run, l
    qh = B[..., 128:192].reshape(B.shape[:-1] + (2, 32))
    q = np.empty(B.shape[:-1] + (2, 4, 32), np.uint8)
    for i in range(4):
        nib = (ql[..., i & 1, :] >> 4) if i >= 2 else (ql[..., i & 1, :] & 15)
        q[..., i, :] = nib | (((qh >> (2 * i)) & 3) << 4)
    return q.reshape(B.shape[:-1] + (256,))


def _q6k_from_codes(q, B):
    q = q.reshape(q.shape[:-1] + (2, 4, 32))
    ql = np.zeros(q.shape[:-3] + (2, 2, 32), np.uint8)
    qh = np.zeros(q.shape[:-3] + (2, 32), np.uint8)
    for i in range(4):
        ql[..., i & 1, :] |= (q[..., i, :] & 15) << (4 if i >= 2 else 0)
        qh |= (q[..., i, :] >> 4) << (2 * i)
    B[..., 0:128] = ql.reshape(q.shape[:-3] + (128,))
    B[..., 128:192] = qh.reshape(q.shape[:-3] + (64,))


def _byte_plane(c):
    """c uint8 [nrt, nb, h, g, 256] (8-bit fields, natural input order) -> bytes [nrt, nb, 4096]."""
    a = c.reshape(c.shape[:4] + (8, 2, 4, 4))                              # P, p, t, b   (s = 2P + p)
    out = a.transpose(0, 1, 4, 3, 6, 5, 2, 7)                               # P, g, t, p, h, b
    return np.ascontiguousarray(out).reshape(out.shape[:2] + (4096,))


def _byte_plane_inv(plane):
    a = plane.reshape(plane.shape[:2] + (8, 8, 4, 2, 2, 4))                # P, g, t, p, h, b
    a = a.transpose(0, 1, 6, 3, 2, 5, 4, 7)                                 # h, g, P, p, t, b
    return np.ascontiguousarray(a).reshape(a.shape[:4] + (256,))


def _q5k_codes(B):
    """[.., 176] -> 5-bit codes [.., 256] in natural input order: element 64G + 32u + l = nibble u of qs[32G + l] | bit 2G + u of qh[l] << 4
    (kyojin_mlx/foreign_gguf.py:470-478)."""
    qh = B[..., 16:48]
    qs = B[..., 48:176].reshape(B.shape[:-1] + (4, 32))
    q = np.empty(B.shape[:-1] + (4, 2, 32), np.uint8)
    for G in range(4):
        for u in range(2):
            nib = (qs[..., G, :] >> 4) if u else (qs[..., G, :] & 15)
            q[..., G, u, :] = nib | (((qh >> (2 * G + u)) & 1) << 4)
    return q.reshape(B.shape[:-1] + (256,))


def _q5k_from_codes(q, B):
    q = q.reshape(q.shape[:-1] + (4, 2, 32))
    qs = np.zeros(q.shape[:-3] + (4, 32), np.uint8)
    qh = np.zeros(q.shape[:-3] + (32,), np.uint8)
    for G in range(4):
        for u in range(2):
            qs[..., G, :] |= (q[..., G, u, :] & 15) << (4 * u)
            qh |= (q[..., G, u, :] >> 4) << (2 * G + u)
    B[..., 16:48] = qh
    B[..., 48:176] = qs.reshape(q.shape[:-3] + (128,))


def _q3k_codes(B):
    """[.., 110] -> (2-bit codes, high bits) [.., 256] each, natural input order (foreign_gguf.py:551-555)."""
    hm = B[..., 0:32]
    qs = B[..., 32:96].reshape(B.shape[:-1] + (2, 32))
    lo = np.empty(B.shape[:-1] + (2, 4, 32), np.uint8)
    hb = np.empty_like(lo)
    for h in range(2):
        for j in range(4):
            lo[..., h, j, :] = (qs[..., h, :] >> (2 * j)) & 3
            hb[..., h, j, :] = (hm >> (4 * h + j)) & 1
    return lo.reshape(B.shape[:-1] + (256,)), hb.reshape(B.shape[:-1] + (256,))


def _q3k_from_codes(lo, hb, B):
    lo = lo.reshape(lo.shape[:-1] + (2, 4, 32))
    hb = hb.reshape(hb.shape[:-1] + (2, 4, 32))
    qs = np.zeros(lo.shape[:-3] + (2, 32), np.uint8)
    hm = np.zeros(lo.shape[:-3] + (32,), np.uint8)
    for h in range(2):
        for j in range(4):
            qs[..., h, :] |= lo[..., h, j, :] << (2 * j)
            hm |= hb[..., h, j, :] << (4 * h + j)
    B[..., 0:32] = hm
    B[..., 32:96] = qs.reshape(lo.shape[:-3] + (64,))


def nvfp4_raw_to_codes(raw, k):
    """GGUF NVFP4 rows -> (codes uint8 [n, k] natural order, scale bytes uint8 [n, k/16]). (foreign_gguf.py:688-692)"""
    raw = np.asarray(raw, np.uint8)
    n = raw.shape[0]
    B = raw.reshape(n, k // 64, 36)
    q = B[..., 4:36].reshape(n, k // 64, 4, 8)
    codes = np.concatenate([q & 15, q >> 4], -1).reshape(n, k)
    return codes, np.ascontiguousarray(B[..., 0:4]).reshape(n, k // 16)


def nvfp4_codes_to_raw(codes, scales):
    n, k = codes.shape
    c = codes.reshape(n, k // 64, 4, 2, 8)
    B = np.empty((n, k // 64, 36), np.uint8)
    B[..., 0:4] = scales.reshape(n, k // 64, 4)
    B[..., 4:36] = (c[..., 0, :] | (c[..., 1, :] << 4)).reshape(n, k // 64, 32)
    return B.reshape(n, -1)


def nvfp4_pack_to_codes(qs, meta):
    """pack form (qs uint8 [n, k/2]: byte b = input 2b | input 2b+1 << 4; meta uint16 [n, k/32]) -> (codes, scale bytes).
    (kyojin_mlx/foreign_pack.py:209-211)"""
    qs = np.asarray(qs, np.uint8)
    n, k = qs.shape[0], qs.shape[1] * 2
    codes = np.empty((n, k), np.uint8)
    codes[:, 0::2], codes[:, 1::2] = qs & 15, qs >> 4
    return codes, np.ascontiguousarray(meta).view(np.uint8).reshape(n, k // 16)


def nvfp4_codes_to_pack(codes, scales):
    n, k = codes.shape
    return np.ascontiguousarray(codes[:, 0::2] | (codes[:, 1::2] << 4)), np.ascontiguousarray(scales).view("<u2").reshape(n, k // 32)


def raw_to_t16(fmt: str, raw, n: int, k: int) -> np.ndarray:
    """GGUF rows uint8 [n, row_bytes] -> T16 bytes uint8 [t16_nbytes]."""
    _check(fmt, k)
    raw = np.asarray(raw, np.uint8)
    if raw.shape != (n, raw_row_bytes(fmt, k)):
        raise ValueError(f"{fmt}: raw {raw.shape} != ({n}, {raw_row_bytes(fmt, k)})")
    nb = k // KBLOCK
    if fmt == "nvfp4":
        codes, sc = nvfp4_raw_to_codes(raw, k)
        return nvfp4_codes_to_t16(codes, sc)
    B = _by_tile(_pad_rows(raw, n).reshape(padded_rows(n), nb, KBLOCK // RAW_BLOCK[fmt][0] * RAW_BLOCK[fmt][1]))           # [nrt, nb, h, g, stored bytes of 256 inputs]
    nrt = B.shape[0]
    if fmt == "q5_k":
        q = _q5k_codes(B)
        parts = [_nibble_plane(q & 15), _onebit_plane(q >> 4), np.ascontiguousarray(B[..., 0:16]).reshape(nrt, nb, 256)]
    elif fmt == "q8_0":
        blk = B.reshape(B.shape[:4] + (8, 34))
        parts = [_byte_plane(np.ascontiguousarray(blk[..., 2:34]).reshape(B.shape[:4] + (256,))), np.ascontiguousarray(blk[..., 0:2]).reshape(nrt, nb, 256)]
    elif fmt == "iq4_xs":
        qs = B[..., 8:136].reshape(B.shape[:-1] + (8, 16))
        codes = np.concatenate([qs & 15, qs >> 4], -1)                                               # [.., sub-block, 32]: element 32 ib + j | 32 ib + 16 + j
        parts = [_nibble_plane(np.ascontiguousarray(codes).reshape(B.shape[:-1] + (256,))), np.ascontiguousarray(B[..., 0:8]).reshape(nrt, nb, 128)]
    elif fmt == "q2_k":
        qs = B[..., 16:80].reshape(B.shape[:-1] + (2, 32))
        lo = np.stack([(qs >> (2 * j)) & 3 for j in range(4)], -2)                                   # [.., half128, j, l]: element 128 h + 32 j + l
        parts = [_twobit_plane(np.ascontiguousarray(lo).reshape(B.shape[:-1] + (256,))), np.ascontiguousarray(B[..., 0:16]).reshape(nrt, nb, 256),
                 np.ascontiguousarray(B[..., 80:84]).reshape(nrt, nb, 64)]
    elif fmt == "q4_k":
        w = np.ascontiguousarray(B[..., 16:144]).view("<u4").reshape(nrt, nb, 2, 8, 4, 2, 4)      # h, g, G, c, t
        quant = np.ascontiguousarray(w.transpose(0, 1, 4, 3, 6, 5, 2)).view(np.uint8).reshape(nrt, nb, 2048)    # G, g, t, c, h
        parts = [quant, np.ascontiguousarray(B[..., 0:16]).reshape(nrt, nb, 256)]
    elif fmt == "q6_k":
        q = _q6k_codes(B)
        parts = [_nibble_plane(q & 15), _twobit_plane(q >> 4), np.ascontiguousarray(B[..., 192:208]).reshape(nrt, nb, 256),
                 np.ascontiguousarray(B[..., 208:210]).reshape(nrt, nb, 32)]
    else:
        lo, hb = _q3k_codes(B)
        parts = [_twobit_plane(lo), _onebit_plane(hb), np.ascontiguousarray(B[..., 96:108]).reshape(nrt, nb, 192),
                 np.ascontiguousarray(B[..., 108:110]).reshape(nrt, nb, 32)]
    return np.ascontiguousarray(np.concatenate(parts, -1)).reshape(-1)


def nvfp4_codes_to_t16(codes, scales) -> np.ndarray:
    n, k = codes.shape
    _check("nvfp4", k)
    nb = k // KBLOCK
    c = _by_tile(_pad_rows(np.asarray(codes, np.uint8), n).reshape(padded_rows(n), nb, 256))
    s = _by_tile(_pad_rows(np.asarray(scales, np.uint8), n).reshape(padded_rows(n), nb, 16))
    nrt = c.shape[0]
    return np.ascontiguousarray(np.concatenate([_fp4_plane(c), np.ascontiguousarray(s).reshape(nrt, nb, 256)], -1)).reshape(-1)


def t16_to_nvfp4_codes(t16, n: int, k: int):
    nb = k // KBLOCK
    T = np.asarray(t16, np.uint8).reshape(padded_rows(n) // ROWS, nb, TILE_BYTES["nvfp4"])
    codes = _from_tile(_fp4_plane_inv(T[..., 0:2048])).reshape(-1, k)[:n]
    sc = _from_tile(T[..., 2048:2304].reshape(T.shape[:2] + (2, 8, 16))).reshape(-1, k // 16)[:n]
    return np.ascontiguousarray(codes), np.ascontiguousarray(sc)


def t16_to_raw(fmt: str, t16, n: int, k: int) -> np.ndarray:
    """Inverse of raw_to_t16 (padding rows dropped): T16 bytes -> GGUF rows uint8 [n, row_bytes]."""
    _check(fmt, k)
    nb = k // KBLOCK
    if fmt == "nvfp4":
        return nvfp4_codes_to_raw(*t16_to_nvfp4_codes(t16, n, k))
    T = np.asarray(t16, np.uint8).reshape(padded_rows(n) // ROWS, nb, TILE_BYTES[fmt])
    nrt = T.shape[0]
    B = np.zeros((nrt, nb, 2, 8, KBLOCK // RAW_BLOCK[fmt][0] * RAW_BLOCK[fmt][1]), np.uint8)
    if fmt == "q5_k":
        _q5k_from_codes(_nibble_plane_inv(T[..., 0:2048]) | (_onebit_plane_inv(T[..., 2048:2560]) << 4), B)
        B[..., 0:16] = T[..., 2560:2816].reshape(nrt, nb, 2, 8, 16)
    elif fmt == "q8_0":
        blk = B.reshape(nrt, nb, 2, 8, 8, 34)
        blk[..., 2:34] = _byte_plane_inv(T[..., 0:4096]).reshape(nrt, nb, 2, 8, 8, 32)
        blk[..., 0:2] = T[..., 4096:4352].reshape(nrt, nb, 2, 8, 8, 2)
    elif fmt == "iq4_xs":
        codes = _nibble_plane_inv(T[..., 0:2048]).reshape(nrt, nb, 2, 8, 8, 2, 16)                   # sub-block, nibble, j
        B[..., 8:136] = (codes[..., 0, :] | (codes[..., 1, :] << 4)).reshape(nrt, nb, 2, 8, 128)
        B[..., 0:8] = T[..., 2048:2176].reshape(nrt, nb, 2, 8, 8)
    elif fmt == "q2_k":
        lo = _twobit_plane_inv(T[..., 0:1024]).reshape(nrt, nb, 2, 8, 2, 4, 32)                    # half128, j, l
        qs = np.zeros((nrt, nb, 2, 8, 2, 32), np.uint8)
        for j in range(4):
            qs |= lo[..., j, :] << (2 * j)
        B[..., 16:80] = qs.reshape(nrt, nb, 2, 8, 64)
        B[..., 0:16] = T[..., 1024:1280].reshape(nrt, nb, 2, 8, 16)
        B[..., 80:84] = T[..., 1280:1344].reshape(nrt, nb, 2, 8, 4)
    elif fmt == "q4_k":
        w = np.ascontiguousarray(T[..., 0:2048]).view("<u4").reshape(nrt, nb, 4, 8, 4, 2, 2)       # G, g, t, c, h
        B[..., 16:144] = np.ascontiguousarray(w.transpose(0, 1, 6, 3, 2, 5, 4)).view(np.uint8).reshape(nrt, nb, 2, 8, 128)
        B[..., 0:16] = T[..., 2048:2304].reshape(nrt, nb, 2, 8, 16)
    elif fmt == "q6_k":
        q = _nibble_plane_inv(T[..., 0:2048]) | (_twobit_plane_inv(T[..., 2048:3072]) << 4)
        _q6k_from_codes(q, B)
        B[..., 192:208] = T[..., 3072:3328].reshape(nrt, nb, 2, 8, 16)
        B[..., 208:210] = T[..., 3328:3360].reshape(nrt, nb, 2, 8, 2)
    else:
        _q3k_from_codes(_twobit_plane_inv(T[..., 0:1024]), _onebit_plane_inv(T[..., 1024:1536]), B)
        B[..., 96:108] = T[..., 1536:1728].reshape(nrt, nb, 2, 8, 12)
        B[..., 108:110] = T[..., 1728:1760].reshape(nrt, nb, 2, 8, 2)
    return np.ascontiguousarray(_from_tile(B).reshape(nrt * ROWS, -1)[:n])
