"""numpy restatement of the reference's block decoders and of the dequant-then-matmul path.

TEST INFRASTRUCTURE (see oracle/__init__.py). Each function cites the reference lines it follows.
All scale arithmetic is float32 in the reference's association order, so results are bit-equal to
the reference decoder (checked by tests/test_oracle_golden.py against committed fixtures).
"""
from __future__ import annotations

import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np

# block elements / block bytes (kyojin_mlx/foreign_gguf.py:27-35 TYPES)
BLOCK = {"Q4_K": (256, 144), "Q3_K": (256, 110), "Q6_K": (256, 210), "NVFP4": (64, 36), "Q5_K": (256, 176), "Q8_0": (32, 34), "Q2_K": (256, 84), "IQ4_XS": (256, 136)}

# doubled e2m1 magnitudes used with the halved scale of GGUF NVFP4 (foreign_gguf.py:69)
_FP4_X2 = np.array([0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12], np.float32)
# plain e2m1 values of the pack form (foreign_pack.py:22)
_E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], np.float32)


def row_bytes(tname: str, k: int) -> int:
    be, bb = BLOCK[tname]
    if k % be:
        raise ValueError(f"{tname}: k={k} is not a multiple of {be}")
    return k // be * bb


def _half_field(blocks: np.ndarray, at: int) -> np.ndarray:
    """fp16 field at byte offset `at` of every block -> float32 [..]. (foreign_gguf.py:331-332)"""
    return np.ascontiguousarray(blocks[..., at:at + 2]).view("<f2")[..., 0].astype(np.float32)


def k4_scales_mins(s12: np.ndarray):
    """12 packed bytes -> (scale[8], min[8]) uint8, the 6-bit fields of Q4_K. (foreign_gguf.py:340-346)"""
    s12 = np.asarray(s12, np.uint8)
    sc = np.zeros(s12.shape[:-1] + (8,), np.uint8)
    mn = np.zeros_like(sc)
    for j in range(4):
        sc[..., j] = s12[..., j] & 63
        mn[..., j] = s12[..., j + 4] & 63
        sc[..., j + 4] = (s12[..., j + 8] & 15) | ((s12[..., j] >> 6) << 4)
        mn[..., j + 4] = (s12[..., j + 8] >> 4) | ((s12[..., j + 4] >> 6) << 4)
    return sc, mn


def q3_scales(s12: np.ndarray) -> np.ndarray:
    """12 packed bytes -> 16 six-bit scales (still biased by +32), Q3_K. (foreign_gguf.py:545-550)"""
    s12 = np.asarray(s12, np.uint8)
    out = np.zeros(s12.shape[:-1] + (16,), np.uint8)
    for j in range(4):
        top = s12[..., 8 + j]
        out[..., j] = (s12[..., j] & 15) | ((top & 3) << 4)
        out[..., j + 4] = (s12[..., j + 4] & 15) | (((top >> 2) & 3) << 4)
        out[..., j + 8] = (s12[..., j] >> 4) | (((top >> 4) & 3) << 4)
        out[..., j + 12] = (s12[..., j + 4] >> 4) | (((top >> 6) & 3) << 4)
    return out


def ue4m3_half(b: np.ndarray) -> np.ndarray:
    """GGUF NVFP4 scale byte -> float32 of HALF the e4m3 value; 0x00 and 0x7F give 0.
    (foreign_gguf.py:349-354 with the * 0.5 of :458)"""
    b = np.asarray(b, np.uint8)
    e = ((b >> 3) & 15).astype(np.int32)
    m = (b & 7).astype(np.float32)
    v = np.where(e == 0, np.ldexp(m, -9), np.ldexp(np.float32(1.0) + m / np.float32(8.0), e - 7)).astype(np.float32)
    v = np.where((b == 0) | (b == 0x7F), np.float32(0.0), v).astype(np.float32)
    return v * np.float32(0.5)


def e4m3_unsigned(b: np.ndarray) -> np.ndarray:
    """pack-form NVFP4 scale byte: sign bit ignored, 0x7F -> 0. (foreign_pack.py:113-117)"""
    b = np.asarray(b, np.uint8) & 127
    e = (b >> 3).astype(np.int32)
    m = (b & 7).astype(np.float32)
    v = np.where(e == 0, np.ldexp(m, -9), np.ldexp(np.float32(1.0) + m / np.float32(8.0), e - 7)).astype(np.float32)
    return np.where(b == 127, np.float32(0.0), v).astype(np.float32)


def _decode_q4k(B):
    """[nr, nb, 144] -> [nr, nb, 256] float32: w = (d*sc)*q - dmin*mn. (foreign_gguf.py:462-469)"""
    d = _half_field(B, 0)[..., None]
    dmin = _half_field(B, 2)[..., None]
    sc, mn = k4_scales_mins(B[..., 4:16])
    q = B[..., 16:144].reshape(B.shape[:-1] + (4, 32))
    out = np.empty(B.shape[:-1] + (8, 32), np.float32)
    for j in range(8):
        nib = (q[..., j // 2, :] >> 4) if (j & 1) else (q[..., j // 2, :] & 15)
        out[..., j, :] = (d * sc[..., j:j + 1].astype(np.float32)) * nib.astype(np.float32) - dmin * mn[..., j:j + 1].astype(np.float32)
    return out.reshape(B.shape[:-1] + (256,))


def _decode_q6k(B):
    """[nr, nb, 210] -> [nr, nb, 256]: w = (d*sc)*(q-32), q = low nibble | 2 high bits << 4. (foreign_gguf.py:481-493)"""
    ql = B[..., 0:128].reshape(B.shape[:-1] + (2, 64))
    qh = B[..., 128:192].reshape(B.shape[:-1] + (2, 32))
    sc = B[..., 192:208].view(np.int8).astype(np.float32)                       # [.., 16]
    d = _half_field(B, 208)[..., None]
    out = np.empty(B.shape[:-1] + (2, 4, 32), np.float32)
    for h in range(2):
        for i in range(4):
            lo = ql[..., h, 32 * (i & 1):32 * (i & 1) + 32]
            nib = (lo >> 4) if i >= 2 else (lo & 15)
            q = (nib | (((qh[..., h, :] >> (2 * i)) & 3) << 4)).astype(np.float32) - np.float32(32.0)
            for c in range(2):                                                    # one scale per 16 elements
                s = sc[..., 8 * h + 2 * i + c][..., None]
                out[..., h, i, 16 * c:16 * c + 16] = (d * s) * q[..., 16 * c:16 * c + 16]
    return out.reshape(B.shape[:-1] + (256,))


def _decode_q3k(B):
    """[nr, nb, 110] -> [nr, nb, 256]: w = (d*(sc-32)) * (2-bit code - (hbit ? 0 : 4)). (foreign_gguf.py:545-557)"""
    hm = B[..., 0:32]
    qs = B[..., 32:96].reshape(B.shape[:-1] + (2, 32))
    sc = q3_scales(B[..., 96:108]).astype(np.int32) - 32
    d = _half_field(B, 108)[..., None]
    out = np.empty(B.shape[:-1] + (2, 4, 32), np.float32)
    for h in range(2):
        for j in range(4):
            code = ((qs[..., h, :] >> (2 * j)) & 3).astype(np.int32)
            hb = (hm >> (4 * h + j)) & 1
            q = (code - np.where(hb != 0, 0, 4)).astype(np.float32)
            for c in range(2):
                dl = d * sc[..., 8 * h + 2 * j + c][..., None].astype(np.float32)
                out[..., h, j, 16 * c:16 * c + 16] = dl * q[..., 16 * c:16 * c + 16]
    return out.reshape(B.shape[:-1] + (256,))


def _decode_nvfp4(B):
    """[nr, nb, 36] -> [nr, nb, 64]: byte j of a 16-sub-block = element j (low) and j+8 (high). (foreign_gguf.py:457-461)"""
    sc = ue4m3_half(B[..., 0:4])                                                  # [.., 4]
    q = B[..., 4:36].reshape(B.shape[:-1] + (4, 8))
    v = np.concatenate([_FP4_X2[q & 15], _FP4_X2[q >> 4]], -1)                   # [.., 4, 16]
    return (v * sc[..., None]).reshape(B.shape[:-1] + (64,))


def _decode_q5k(B):
    """[nr, nb, 176] -> [nr, nb, 256]: w = (d*sc)*q - dmin*mn, q = nibble | (bit 2G+u of qh[l]) << 4 for element 64G + 32u + l.
    (foreign_gguf.py:470-480)"""
    d = _half_field(B, 0)[..., None]
    dmin = _half_field(B, 2)[..., None]
    sc, mn = k4_scales_mins(B[..., 4:16])
    qh = B[..., 16:48]
    q = B[..., 48:176].reshape(B.shape[:-1] + (4, 32))
    out = np.empty(B.shape[:-1] + (8, 32), np.float32)
    for j in range(8):
        nib = (q[..., j // 2, :] >> 4) if (j & 1) else (q[..., j // 2, :] & 15)
        code = nib.astype(np.float32) + ((qh >> j) & 1).astype(np.float32) * np.float32(16.0)
        out[..., j, :] = (d * sc[..., j:j + 1].astype(np.float32)) * code - dmin * mn[..., j:j + 1].astype(np.float32)
    return out.reshape(B.shape[:-1] + (256,))


def _decode_q80(B):
    """[nr, nb, 34] -> [nr, nb, 32]: w = int8 * d. (foreign_gguf.py:447-448)"""
    d = _half_field(B, 0)[..., None]
    return np.ascontiguousarray(B[..., 2:34]).view(np.int8).astype(np.float32) * d


def _decode_q2k(B):
    """[nr, nb, 84] -> [nr, nb, 256]: w = (d * (sc & 15)) * code - dmin * (sc >> 4), one scale byte per 16 elements (index 8 * half128 + 2 * j + sub16),
    element 128 h + 32 j + l = bits 2j of qs[32 h + l]. (foreign_gguf.py:538-545)"""
    sc = B[..., 0:16]
    qs = B[..., 16:80].reshape(B.shape[:-1] + (2, 32))
    d = _half_field(B, 80)[..., None]
    dmin = _half_field(B, 82)[..., None]
    out = np.empty(B.shape[:-1] + (2, 4, 32), np.float32)
    for h in range(2):
        for j in range(4):
            q = ((qs[..., h, :] >> (2 * j)) & 3).astype(np.float32)
            for c in range(2):
                s8 = sc[..., 8 * h + 2 * j + c][..., None]
                out[..., h, j, 16 * c:16 * c + 16] = (d * (s8 & 15).astype(np.float32)) * q[..., 16 * c:16 * c + 16] - dmin * (s8 >> 4).astype(np.float32)
    return out.reshape(B.shape[:-1] + (256,))


KVALUES_IQ4NL = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.float32)      # the non-linear 4-bit grid of IQ4_NL / IQ4_XS


def _decode_iq4xs(B):
    """[nr, nb, 136] -> [nr, nb, 256]: w = grid[code] * (d * (ls - 32)); eight 32-element sub-blocks, ls = 4 low bits from scales_l | 2 high bits from scales_h,
    byte j of sub-block ib = element 32 ib + j (low nibble) and 32 ib + 16 + j (high nibble). (foreign_gguf.py:494-502)"""
    d = _half_field(B, 0)[..., None]
    sh = (B[..., 2].astype(np.uint32) | (B[..., 3].astype(np.uint32) << 8))[..., None]
    sl = B[..., 4:8]
    ib = np.arange(8)
    ls = ((sl[..., ib // 2] >> (4 * (ib % 2))) & 15).astype(np.int32) | (((sh >> (2 * ib)) & 3).astype(np.int32) << 4)
    dl = (d * (ls - 32).astype(np.float32))[..., None]
    qs = B[..., 8:136].reshape(B.shape[:-1] + (8, 16))
    y = np.concatenate([KVALUES_IQ4NL[qs & 15], KVALUES_IQ4NL[qs >> 4]], -1) * dl
    return y.reshape(B.shape[:-1] + (256,)).astype(np.float32)


_DECODERS = {"IQ4_XS": _decode_iq4xs, "Q4_K": _decode_q4k, "Q6_K": _decode_q6k, "Q3_K": _decode_q3k, "NVFP4": _decode_nvfp4, "Q5_K": _decode_q5k, "Q8_0": _decode_q80, "Q2_K": _decode_q2k}


def _dequant_chunk(tname, raw2, k):
    be, bb = BLOCK[tname]
    B = np.ascontiguousarray(raw2).reshape(raw2.shape[0], k // be, bb)
    return np.ascontiguousarray(_DECODERS[tname](B).reshape(raw2.shape[0], k), dtype=np.float32)


def dequant(tname: str, raw, k: int, threads: int | None = None) -> np.ndarray:
    """raw uint8 [.., row_bytes] -> float32 [.., k]. Rows are independent; large inputs are decoded in
    row chunks on a thread pool exactly like the reference (foreign_gguf.py:376-394: chunks of 2^22
    elements, min(8, cpu_count) threads), which makes this the timed CPU baseline too."""
    raw = np.asarray(raw, np.uint8)
    if raw.shape[-1] != row_bytes(tname, k):
        raise ValueError(f"{tname}: rows of {raw.shape[-1]} bytes, expected {row_bytes(tname, k)} for k={k}")
    lead = raw.shape[:-1]
    flat = raw.reshape(-1, raw.shape[-1])
    step = max(1, (1 << 22) // k)
    if flat.shape[0] <= step:
        return _dequant_chunk(tname, flat, k).reshape(lead + (k,))
    out = np.empty((flat.shape[0], k), np.float32)

    def work(i):
        out[i:i + step] = _dequant_chunk(tname, flat[i:i + step], k)

    nthr = threads if threads else max(1, min(8, os.cpu_count() or 1))
    with ThreadPoolExecutor(nthr) as ex:
        list(ex.map(work, range(0, flat.shape[0], step)))
    return out.reshape(lead + (k,))


def dequant_nvfp4_pack(qs, meta, gscale=1.0, apply_gscale=True) -> np.ndarray:
    """pack-form NVFP4 (qs uint8 [n, k/2]: byte b = element 2b | element 2b+1 << 4; meta uint16 [n, k/32] = two
    e4m3 bytes; gscale float32 multiplies the result) -> float32 [n, k]. (foreign_pack.py:209-213)"""
    qs = np.asarray(qs, np.uint8)
    n, k = qs.shape[0], qs.shape[1] * 2
    codes = np.empty((n, k), np.uint8)
    codes[:, 0::2] = qs & 15
    codes[:, 1::2] = qs >> 4
    s = e4m3_unsigned(np.ascontiguousarray(meta).view(np.uint8).reshape(n, k // 16))
    w = (_E2M1[codes].reshape(n, k // 16, 16) * s[..., None]).reshape(n, k)
    return (w * np.float32(gscale)).astype(np.float32) if apply_gscale else w


def nvfp4_gguf_to_pack(raw, k):
    """GGUF NVFP4 rows -> (qs [n, k/2], meta uint16 [n, k/32]) of the pack form, same bits. (foreign_gguf.py:688-692)"""
    raw = np.asarray(raw, np.uint8)
    n = raw.shape[0]
    B = raw.reshape(n, k // 64, 36)
    q = B[..., 4:36].reshape(n, k // 64, 4, 8)
    codes = np.concatenate([q & 15, q >> 4], -1).reshape(n, k)
    qs = np.ascontiguousarray(codes[:, 0::2] | (codes[:, 1::2] << 4))
    sc = np.ascontiguousarray(B[..., 0:4]).reshape(n, k // 16)
    return qs, np.ascontiguousarray(sc).view("<u2").reshape(n, k // 32)


# ------------------------------------------------------------------------------------------------ matmul references
def matmul_f64(x, w32) -> np.ndarray:
    """fp64 dequant-then-matmul, the accuracy reference (tests/test_foreign_formats.py:330)."""
    return np.asarray(x).astype(np.float64) @ np.asarray(w32).astype(np.float64).T


def sat_f16(a) -> np.ndarray:
    """float -> fp16 saturated at +-65504, never inf (foreign_metal.py:344, :1076)."""
    return np.clip(np.asarray(a, np.float32), -65504.0, 65504.0).astype(np.float16)


def matmul_ref_path(x16, w32) -> np.ndarray:
    """CPU restatement of the reference's device arithmetic for a large-row linear: weights rounded to fp16
    (foreign_metal.py:1130-1146 dequant to half), fp16 x, float32 accumulate, saturated fp16 output
    (foreign_linear.py:710 `x2 @ self.dequant().T`). Used for the '<= 2x the reference path's own error' bound."""
    w16 = np.asarray(w32, np.float32).astype(np.float16).astype(np.float32)
    y = np.asarray(x16, np.float16).astype(np.float32) @ w16.T
    return sat_f16(y)


def rel_fro(got, want) -> float:
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    den = np.linalg.norm(want)
    return float(np.linalg.norm(got - want) / den) if den > 0 else float(np.linalg.norm(got - want))


def linear_cpu(tname: str, raw, k: int, x, threads: int | None = None) -> np.ndarray:
    """The reference's CPU path for one linear call: dequantise, then x @ W.T in float32 (arm A of the CPU baseline)."""
    w = dequant(tname, raw, k, threads)
    return np.asarray(x).astype(np.float32) @ w.T
