// Exact decoders of T16 tiles (layout: kyojin_mac_b200/layout.py). Lane L = 4 g + t of a warp owns, for MMA number s of
// a tile, the inputs 16 s + 4 t + b (b = 0..3) of rows g and g + 8. These helpers return the four float32 weights of one
// row with the reference's float32 arithmetic, association order included (kyojin_mlx/foreign_gguf.py:457-557), so the
// dequant kernels are bit-equal to the numpy decoder.
#pragma once
#include "kyb_common.cuh"

namespace kyb {

__device__ __forceinline__ uint32_t ldw(const uint8_t* p) { return *reinterpret_cast<const uint32_t*>(p); }
__device__ __forceinline__ float ldh(const uint8_t* p) { return __half2float(*reinterpret_cast<const __half*>(p)); }

// 6-bit scale / min number j (0..7) of a Q4_K block from its 12 packed bytes (foreign_gguf.py:340-346)
__device__ __forceinline__ void q4k_scale_min(const uint8_t* s12, int j, int& sc, int& mn) {
    if (j < 4) {
        sc = s12[j] & 63;
        mn = s12[j + 4] & 63;
    } else {
        sc = (s12[j + 4] & 15) | ((s12[j - 4] >> 6) << 4);
        mn = (s12[j + 4] >> 4) | ((s12[j] >> 6) << 4);
    }
}

// 6-bit scale number s (0..15) of a Q3_K block, still biased by +32 (foreign_gguf.py:545-550)
__device__ __forceinline__ int q3k_scale(const uint8_t* s12, int s) {
    const int j = s & 3, grp = s >> 2;
    const int lo = s12[(grp & 1) * 4 + j];
    const int nib = (grp & 2) ? (lo >> 4) : (lo & 15);
    return nib | (((s12[8 + j] >> (2 * grp)) & 3) << 4);
}

// e4m3 magnitude of the low 7 bits, 0x7F -> 0 (foreign_pack.py:113-117). Exact: (bits << 20) reinterpreted is value * 2^-120.
__device__ __forceinline__ float e4m3_unsigned(uint32_t b) {
    b &= 127u;
    const float v = __uint_as_float(b << 20) * 1.329227995784916e36f;   // * 2^120
    return b == 127u ? 0.0f : v;
}

__device__ __forceinline__ float e2m1_value(uint32_t code) {
    // 0, .5, 1, 1.5, 2, 3, 4, 6 with sign bit 3: fp16 bits (sign << 15 | mag << 9) are the value * 2^-14
    const uint32_t hb = ((code & 8u) << 12) | ((code & 7u) << 9);
    return half_bits_to_float(hb) * 16384.0f;
}

template <int FMT>
struct TileDecode;

// integer code of input e (0..255) of row r (0..15) of a tile: q4_k nibble, q6_k 6-bit value, q3_k (2-bit | hbit << 2), nvfp4 e2m1 nibble
template <int FMT>
__device__ __forceinline__ uint32_t tile_code(const uint8_t* tile, int r, int e) {
    const int s = e >> 4, t = (e >> 2) & 3, b = e & 3, g = r & 7, h = r >> 3, L = g * 4 + t;
    if (FMT == KYB_FMT_Q4_K) {
        const int j = s >> 1, c = s & 1, G = j >> 1;
        const uint32_t byte = tile[(G * 32 + L) * 16 + (2 * c + h) * 4 + b];
        return (j & 1) ? (byte >> 4) : (byte & 15u);
    } else if (FMT == KYB_FMT_Q6_K) {
        const uint32_t nb = tile[((s >> 2) * 32 + L) * 16 + (2 * ((s >> 1) & 1) + h) * 4 + b];
        const uint32_t hb = tile[2048 + ((s >> 3) * 32 + L) * 16 + (2 * ((s >> 2) & 1) + h) * 4 + b];
        return ((s & 1) ? (nb >> 4) : (nb & 15u)) | (((hb >> (2 * (s & 3))) & 3u) << 4);
    } else if (FMT == KYB_FMT_Q3_K) {
        const uint32_t lb = tile[((s >> 3) * 32 + L) * 16 + (2 * ((s >> 2) & 1) + h) * 4 + b];
        const uint32_t hb = tile[1024 + L * 16 + (2 * (s >> 3) + h) * 4 + b];
        return ((lb >> (2 * (s & 3))) & 3u) | (((hb >> (s & 7)) & 1u) << 2);
    } else if (FMT == KYB_FMT_Q5_K) {
        const uint32_t nb = tile[((s >> 2) * 32 + L) * 16 + (2 * ((s >> 1) & 1) + h) * 4 + b];
        const uint32_t hb = tile[2048 + L * 16 + (2 * (s >> 3) + h) * 4 + b];
        return ((s & 1) ? (nb >> 4) : (nb & 15u)) | (((hb >> (s & 7)) & 1u) << 4);
    } else if (FMT == KYB_FMT_Q8_0) {
        return tile[((s >> 1) * 32 + L) * 16 + (2 * (s & 1) + h) * 4 + b];
    } else if (FMT == KYB_FMT_Q2_K) {
        const uint32_t lb = tile[((s >> 3) * 32 + L) * 16 + (2 * ((s >> 2) & 1) + h) * 4 + b];
        return (lb >> (2 * (s & 3))) & 3u;
    } else if (FMT == KYB_FMT_IQ4_XS) {
        const uint32_t nb = tile[((s >> 2) * 32 + L) * 16 + (2 * ((s >> 1) & 1) + h) * 4 + b];
        return (s & 1) ? (nb >> 4) : (nb & 15u);
    } else {
        const uint32_t word = ldw(tile + ((s >> 2) * 32 + L) * 16 + (2 * ((s >> 1) & 1) + h) * 4);
        const int v = 2 * (s & 1) + (b & 1), j = b >> 1;
        const int mag_at = 9 - 3 * v, sign_at = (v == 0 ? 15 : 11 + v);
        return ((word >> (mag_at + 16 * j)) & 7u) | (((word >> (sign_at + 16 * j)) & 1u) << 3);
    }
}

template <>
struct TileDecode<KYB_FMT_Q4_K> {
    // w[b] = (d * sc) * q - dmin * mn
    static __device__ __forceinline__ void row4(const uint8_t* tile, int g, int t, int h, int s, float gscale, float (&w)[4]) {
        const int j = s >> 1, c = s & 1, G = j >> 1;
        const uint32_t word = ldw(tile + (G * 32 + g * 4 + t) * 16 + (2 * c + h) * 4);
        const uint8_t* meta = tile + 2048 + (g + 8 * h) * 16;
        const float d = ldh(meta), dmin = ldh(meta + 2);
        int sc, mn;
        q4k_scale_min(meta + 4, j, sc, mn);
        const float ds = __fmul_rn(d, (float)sc), dm = __fmul_rn(dmin, (float)mn);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const uint32_t byte = (word >> (8 * b)) & 255u;
            const float q = (float)((j & 1) ? (byte >> 4) : (byte & 15u));
            w[b] = __fsub_rn(__fmul_rn(ds, q), dm);
        }
    }
};

template <>
struct TileDecode<KYB_FMT_Q6_K> {
    // w[b] = (d * sc) * (q - 32)
    static __device__ __forceinline__ void row4(const uint8_t* tile, int g, int t, int h, int s, float gscale, float (&w)[4]) {
        const int L = g * 4 + t;
        const uint32_t nibw = ldw(tile + ((s >> 2) * 32 + L) * 16 + (2 * ((s >> 1) & 1) + h) * 4);
        const uint32_t hiw = ldw(tile + 2048 + ((s >> 3) * 32 + L) * 16 + (2 * ((s >> 2) & 1) + h) * 4);
        const int r = g + 8 * h;
        const float sc = (float)(int)(*reinterpret_cast<const int8_t*>(tile + 3072 + r * 16 + s));
        const float ds = __fmul_rn(ldh(tile + 3328 + r * 2), sc);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const uint32_t nb = (nibw >> (8 * b)) & 255u, hb = (hiw >> (8 * b)) & 255u;
            const int q = (int)(((s & 1) ? (nb >> 4) : (nb & 15u)) | (((hb >> (2 * (s & 3))) & 3u) << 4)) - 32;
            w[b] = __fmul_rn(ds, (float)q);
        }
    }
};

template <>
struct TileDecode<KYB_FMT_Q3_K> {
    // w[b] = (d * (sc - 32)) * (code - (hbit ? 0 : 4))
    static __device__ __forceinline__ void row4(const uint8_t* tile, int g, int t, int h, int s, float gscale, float (&w)[4]) {
        const int L = g * 4 + t;
        const uint32_t low = ldw(tile + ((s >> 3) * 32 + L) * 16 + (2 * ((s >> 2) & 1) + h) * 4);
        const uint32_t hbw = ldw(tile + 1024 + L * 16 + (2 * (s >> 3) + h) * 4);
        const int r = g + 8 * h;
        const int sc = q3k_scale(tile + 1536 + r * 12, s) - 32;
        const float dl = __fmul_rn(ldh(tile + 1728 + r * 2), (float)sc);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const uint32_t lb = (low >> (8 * b)) & 255u, hb = (hbw >> (8 * b)) & 255u;
            const int q = (int)((lb >> (2 * (s & 3))) & 3u) - (((hb >> (s & 7)) & 1u) ? 0 : 4);
            w[b] = __fmul_rn(dl, (float)q);
        }
    }
};

template <>
struct TileDecode<KYB_FMT_Q5_K> {
    // w[b] = (d * sc) * q - dmin * mn, q = 4-bit code | high bit << 4 (kyojin_mlx/foreign_gguf.py:470-480)
    static __device__ __forceinline__ void row4(const uint8_t* tile, int g, int t, int h, int s, float gscale, float (&w)[4]) {
        const uint8_t* meta = tile + 2560 + (g + 8 * h) * 16;
        const float d = ldh(meta), dmin = ldh(meta + 2);
        int sc, mn;
        q4k_scale_min(meta + 4, s >> 1, sc, mn);
        const float ds = __fmul_rn(d, (float)sc), dm = __fmul_rn(dmin, (float)mn);
#pragma unroll
        for (int b = 0; b < 4; ++b) w[b] = __fsub_rn(__fmul_rn(ds, (float)tile_code<KYB_FMT_Q5_K>(tile, g + 8 * h, 16 * s + 4 * t + b)), dm);
    }
};

template <>
struct TileDecode<KYB_FMT_Q8_0> {
    // w[b] = q * d with one fp16 d per 32 inputs (kyojin_mlx/foreign_gguf.py:447-448)
    static __device__ __forceinline__ void row4(const uint8_t* tile, int g, int t, int h, int s, float gscale, float (&w)[4]) {
        const int r = g + 8 * h;
        const float d = ldh(tile + 4096 + r * 16 + (s >> 1) * 2);
#pragma unroll
        for (int b = 0; b < 4; ++b) w[b] = __fmul_rn((float)(int)(int8_t)tile_code<KYB_FMT_Q8_0>(tile, r, 16 * s + 4 * t + b), d);
    }
};

// the non-linear 4-bit grid of IQ4_NL / IQ4_XS (kyojin_mlx/foreign_gguf.py:68), as four little-endian words of int8
__device__ __forceinline__ float iq4nl_value(uint32_t code) {
    const uint32_t w = code < 4 ? 0xBFAD9881u : code < 8 ? 0xF6EADDCFu : code < 12 ? 0x26190D01u : 0x71594535u;
    return (float)(int)(int8_t)((w >> (8 * (code & 3u))) & 255u);
}
// 6-bit scale of sub-block ib (0..7) of an IQ4_XS block, still biased by +32: 4 low bits from scales_l, 2 high bits from scales_h (foreign_gguf.py:494-500)
__device__ __forceinline__ int iq4xs_scale(const uint8_t* meta, int ib) {
    const uint32_t sh = (uint32_t)meta[2] | ((uint32_t)meta[3] << 8);
    return (int)(((meta[4 + (ib >> 1)] >> (4 * (ib & 1))) & 15u) | (((sh >> (2 * ib)) & 3u) << 4));
}

template <>
struct TileDecode<KYB_FMT_IQ4_XS> {
    // w[b] = grid[code] * (d * (ls - 32))
    static __device__ __forceinline__ void row4(const uint8_t* tile, int g, int t, int h, int s, float gscale, float (&w)[4]) {
        const int r = g + 8 * h;
        const uint8_t* meta = tile + 2048 + r * 8;
        const float dl = __fmul_rn(ldh(meta), (float)(iq4xs_scale(meta, s >> 1) - 32));
#pragma unroll
        for (int b = 0; b < 4; ++b) w[b] = __fmul_rn(iq4nl_value(tile_code<KYB_FMT_IQ4_XS>(tile, r, 16 * s + 4 * t + b)), dl);
    }
};

template <>
struct TileDecode<KYB_FMT_Q2_K> {
    // w[b] = (d * (sc & 15)) * code - dmin * (sc >> 4), one scale byte per 16 inputs (kyojin_mlx/foreign_gguf.py:538-545)
    static __device__ __forceinline__ void row4(const uint8_t* tile, int g, int t, int h, int s, float gscale, float (&w)[4]) {
        const int r = g + 8 * h;
        const uint32_t sb = tile[1024 + r * 16 + s];
        const float ds = __fmul_rn(ldh(tile + 1280 + r * 4), (float)(sb & 15u)), dm = __fmul_rn(ldh(tile + 1280 + r * 4 + 2), (float)(sb >> 4));
#pragma unroll
        for (int b = 0; b < 4; ++b) w[b] = __fsub_rn(__fmul_rn(ds, (float)tile_code<KYB_FMT_Q2_K>(tile, r, 16 * s + 4 * t + b)), dm);
    }
};

template <>
struct TileDecode<KYB_FMT_NVFP4> {
    // w[b] = (e2m1 * e4m3 scale) * gscale
    static __device__ __forceinline__ void row4(const uint8_t* tile, int g, int t, int h, int s, float gscale, float (&w)[4]) {
        const int L = g * 4 + t;
        const uint32_t word = ldw(tile + ((s >> 2) * 32 + L) * 16 + (2 * ((s >> 1) & 1) + h) * 4);
        const int r = g + 8 * h;
        const float sc = e4m3_unsigned(tile[2048 + r * 16 + s]);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int v = 2 * (s & 1) + (b & 1), j = b >> 1;
            const int mag_at = 9 - 3 * v, sign_at = (v == 0 ? 15 : 11 + v);
            const uint32_t code = ((word >> (mag_at + 16 * j)) & 7u) | (((word >> (sign_at + 16 * j)) & 1u) << 3);
            w[b] = __fmul_rn(__fmul_rn(e2m1_value(code), sc), gscale);
        }
    }
};

}  // namespace kyb
