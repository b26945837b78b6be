// Load-time repack between stored GGUF rows and the T16 layout, on the device (a pure bit permutation; the numpy twin is
// kyojin_mac_b200/layout.py). One thread builds one 32-bit word of the destination.
#include "t16_decode.cuh"

namespace kyb {

// ---- codes of a stored 256-input super-block (for NVFP4: four consecutive 36-byte blocks)
template <int FMT>
__device__ __forceinline__ uint32_t raw_code(const uint8_t* blk, int e) {
    if (FMT == KYB_FMT_Q4_K) {                       // byte l of 64-group G: input 64G+l (low), 64G+32+l (high)
        const uint32_t byte = blk[16 + (e >> 6) * 32 + (e & 31)];
        return (e & 32) ? (byte >> 4) : (byte & 15u);
    } else if (FMT == KYB_FMT_Q6_K) {                // input 128H + 32i + l: ql[64H + 32(i&1) + l] nibble (i>=2: high), qh[32H + l] bits 2i
        const int H = e >> 7, i = (e >> 5) & 3, l = e & 31;
        const uint32_t lo = blk[64 * H + 32 * (i & 1) + l], hi = blk[128 + 32 * H + l];
        return ((i & 2) ? (lo >> 4) : (lo & 15u)) | (((hi >> (2 * i)) & 3u) << 4);
    } else if (FMT == KYB_FMT_Q3_K) {                // input 128H + 32j + l: qs[32H + l] bits 2j, hmask[l] bit 4H + j
        const int H = e >> 7, j = (e >> 5) & 3, l = e & 31;
        return ((blk[32 + 32 * H + l] >> (2 * j)) & 3u) | (((blk[l] >> (4 * H + j)) & 1u) << 2);
    } else if (FMT == KYB_FMT_Q5_K) {                // as Q4_K behind the 32 bytes of high bits: bit e / 32 of qh[e % 32]
        const uint32_t byte = blk[48 + (e >> 6) * 32 + (e & 31)];
        return ((e & 32) ? (byte >> 4) : (byte & 15u)) | (((blk[16 + (e & 31)] >> (e >> 5)) & 1u) << 4);
    } else if (FMT == KYB_FMT_Q8_0) {                // eight 34-byte blocks: fp16 d, 32 int8
        return blk[34 * (e >> 5) + 2 + (e & 31)];
    } else if (FMT == KYB_FMT_IQ4_XS) {              // sub-block ib of 32: byte j of its 16 = input 32 ib + j (low nibble), 32 ib + 16 + j (high), behind 8 bytes of d / scales
        const uint32_t byte = blk[8 + 16 * (e >> 5) + (e & 15)];
        return (e & 16) ? (byte >> 4) : (byte & 15u);
    } else if (FMT == KYB_FMT_Q2_K) {                // input 128H + 32j + l: qs[32H + l] bits 2j, behind the 16 scale bytes
        const int H = e >> 7, j = (e >> 5) & 3, l = e & 31;
        return (blk[16 + 32 * H + l] >> (2 * j)) & 3u;
    } else {                                         // 64-block B, 16-sub-block u, l: byte 4 + 8u + (l & 7), nibble l >> 3
        const int B = e >> 6, u = (e >> 4) & 3, l = e & 15;
        const uint32_t byte = blk[36 * B + 4 + 8 * u + (l & 7)];
        return (l & 8) ? (byte >> 4) : (byte & 15u);
    }
}

template <int FMT>
__global__ void raw_to_t16_kernel(const uint8_t* __restrict__ raw, int64_t n, int64_t nb, uint8_t* __restrict__ t16, int64_t total_words) {
    constexpr int TB = kyb_tile_bytes(FMT), TW = TB / 4;
    constexpr int RB = kyb_raw_kblock_bytes(FMT);                                     // stored bytes of one 256-input block
    const int64_t gw = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gw >= total_words) return;
    const int64_t tile = gw / TW;
    const int wi = (int)(gw % TW);
    const int64_t rt = tile / nb, kb = tile % nb;
    uint32_t out = 0;
    auto blk_of = [&](int r) -> const uint8_t* {
        const int64_t row = rt * 16 + r;
        return row < n ? raw + (row * nb + kb) * RB : nullptr;
    };
    auto unit = [&](int widx, int& P, int& g, int& t, int& a, int& h) {   // word `widx` of a [P][lane][4 words] plane
        P = widx >> 7;
        const int L = (widx >> 2) & 31;
        g = L >> 2, t = L & 3, a = (widx >> 1) & 1, h = widx & 1;
    };
    int P, g, t, a, h;
    if (FMT == KYB_FMT_Q4_K) {
        if (wi < 512) {
            unit(wi, P, g, t, a, h);
            const uint8_t* b = blk_of(g + 8 * h);
            if (b)
                for (int i = 0; i < 4; ++i) out |= (uint32_t)b[16 + 4 * (8 * P + 4 * a + t) + i] << (8 * i);
        } else {
            const int r = (wi - 512) >> 2, w = (wi - 512) & 3;
            const uint8_t* b = blk_of(r);
            if (b)
                for (int i = 0; i < 4; ++i) out |= (uint32_t)b[4 * w + i] << (8 * i);
        }
    } else if (FMT == KYB_FMT_Q6_K) {
        if (wi < 512) {                              // nibble plane: s0 = 4P + 2a, s1 = s0 + 1
            unit(wi, P, g, t, a, h);
            const uint8_t* b = blk_of(g + 8 * h);
            if (b)
                for (int i = 0; i < 4; ++i) {
                    const int e0 = 16 * (4 * P + 2 * a) + 4 * t + i;
                    out |= ((raw_code<FMT>(b, e0) & 15u) | ((raw_code<FMT>(b, e0 + 16) & 15u) << 4)) << (8 * i);
                }
        } else if (wi < 768) {                       // 2-bit plane: s = 8P + 4a + i2
            unit(wi - 512, P, g, t, a, h);
            const uint8_t* b = blk_of(g + 8 * h);
            if (b)
                for (int i = 0; i < 4; ++i)
                    for (int i2 = 0; i2 < 4; ++i2) out |= (raw_code<FMT>(b, 16 * (8 * P + 4 * a + i2) + 4 * t + i) >> 4) << (8 * i + 2 * i2);
        } else if (wi < 832) {                       // 16 int8 scales per row
            const int r = (wi - 768) >> 2, w = (wi - 768) & 3;
            const uint8_t* b = blk_of(r);
            if (b)
                for (int i = 0; i < 4; ++i) out |= (uint32_t)b[192 + 4 * w + i] << (8 * i);
        } else {                                     // fp16 d, two rows per word
            const int r = (wi - 832) * 2;
            for (int q = 0; q < 2; ++q) {
                const uint8_t* b = blk_of(r + q);
                if (b) out |= ((uint32_t)b[208] | ((uint32_t)b[209] << 8)) << (16 * q);
            }
        }
    } else if (FMT == KYB_FMT_Q3_K) {
        if (wi < 256) {                              // 2-bit plane
            unit(wi, P, g, t, a, h);
            const uint8_t* b = blk_of(g + 8 * h);
            if (b)
                for (int i = 0; i < 4; ++i)
                    for (int i2 = 0; i2 < 4; ++i2) out |= (raw_code<FMT>(b, 16 * (8 * P + 4 * a + i2) + 4 * t + i) & 3u) << (8 * i + 2 * i2);
        } else if (wi < 384) {                       // 1-bit plane: s = 8a + i8
            unit(wi - 256, P, g, t, a, h);
            const uint8_t* b = blk_of(g + 8 * h);
            if (b)
                for (int i = 0; i < 4; ++i)
                    for (int i8 = 0; i8 < 8; ++i8) out |= (raw_code<FMT>(b, 16 * (8 * a + i8) + 4 * t + i) >> 2) << (8 * i + i8);
        } else if (wi < 432) {                       // 12 scale bytes per row = 3 words
            const int r = (wi - 384) / 3, w = (wi - 384) % 3;
            const uint8_t* b = blk_of(r);
            if (b)
                for (int i = 0; i < 4; ++i) out |= (uint32_t)b[96 + 4 * w + i] << (8 * i);
        } else {
            const int r = (wi - 432) * 2;
            for (int q = 0; q < 2; ++q) {
                const uint8_t* b = blk_of(r + q);
                if (b) out |= ((uint32_t)b[108] | ((uint32_t)b[109] << 8)) << (16 * q);
            }
        }
    } else if (FMT == KYB_FMT_Q5_K) {
        if (wi < 512) {                              // nibble plane (low 4 bits of the code): s0 = 4P + 2a, s1 = s0 + 1
            unit(wi, P, g, t, a, h);
            const uint8_t* b = blk_of(g + 8 * h);
            if (b)
                for (int i = 0; i < 4; ++i) {
                    const int e0 = 16 * (4 * P + 2 * a) + 4 * t + i;
                    out |= ((raw_code<FMT>(b, e0) & 15u) | ((raw_code<FMT>(b, e0 + 16) & 15u) << 4)) << (8 * i);
                }
        } else if (wi < 640) {                       // 1-bit plane (the fifth bit): s = 8a + i8
            unit(wi - 512, P, g, t, a, h);
            const uint8_t* b = blk_of(g + 8 * h);
            if (b)
                for (int i = 0; i < 4; ++i)
                    for (int i8 = 0; i8 < 8; ++i8) out |= (raw_code<FMT>(b, 16 * (8 * a + i8) + 4 * t + i) >> 4) << (8 * i + i8);
        } else {                                     // d, dmin, 12 scale bytes of every row
            const int r = (wi - 640) >> 2, w = (wi - 640) & 3;
            const uint8_t* b = blk_of(r);
            if (b)
                for (int i = 0; i < 4; ++i) out |= (uint32_t)b[4 * w + i] << (8 * i);
        }
    } else if (FMT == KYB_FMT_IQ4_XS) {
        if (wi < 512) {                              // nibble plane: s0 = 4P + 2a, s1 = s0 + 1
            unit(wi, P, g, t, a, h);
            const uint8_t* b = blk_of(g + 8 * h);
            if (b)
                for (int i = 0; i < 4; ++i) {
                    const int e0 = 16 * (4 * P + 2 * a) + 4 * t + i;
                    out |= (raw_code<FMT>(b, e0) | (raw_code<FMT>(b, e0 + 16) << 4)) << (8 * i);
                }
        } else {                                     // d, scales_h, scales_l of every row: 2 words
            const int r = (wi - 512) >> 1, w = (wi - 512) & 1;
            const uint8_t* b = blk_of(r);
            if (b)
                for (int i = 0; i < 4; ++i) out |= (uint32_t)b[4 * w + i] << (8 * i);
        }
    } else if (FMT == KYB_FMT_Q2_K) {
        if (wi < 256) {                              // 2-bit plane (as Q3_K)
            unit(wi, P, g, t, a, h);
            const uint8_t* b = blk_of(g + 8 * h);
            if (b)
                for (int i = 0; i < 4; ++i)
                    for (int i2 = 0; i2 < 4; ++i2) out |= raw_code<FMT>(b, 16 * (8 * P + 4 * a + i2) + 4 * t + i) << (8 * i + 2 * i2);
        } else if (wi < 320) {                       // 16 scale | min bytes per row = 4 words
            const int r = (wi - 256) >> 2, w = (wi - 256) & 3;
            const uint8_t* b = blk_of(r);
            if (b)
                for (int i = 0; i < 4; ++i) out |= (uint32_t)b[4 * w + i] << (8 * i);
        } else {                                     // fp16 d, fp16 dmin of one row
            const uint8_t* b = blk_of(wi - 320);
            if (b)
                for (int i = 0; i < 4; ++i) out |= (uint32_t)b[80 + i] << (8 * i);
        }
    } else if (FMT == KYB_FMT_Q8_0) {
        if (wi < 1024) {                             // byte plane: unit P holds slices 2P (a = 0) and 2P + 1 (a = 1)
            unit(wi, P, g, t, a, h);
            const uint8_t* b = blk_of(g + 8 * h);
            if (b)
                for (int i = 0; i < 4; ++i) out |= raw_code<FMT>(b, 16 * (2 * P + a) + 4 * t + i) << (8 * i);
        } else {                                     // eight fp16 d per row, two per word
            const int r = (wi - 1024) >> 2, w = (wi - 1024) & 3;
            const uint8_t* b = blk_of(r);
            if (b)
                for (int q = 0; q < 2; ++q) out |= ((uint32_t)b[34 * (2 * w + q)] | ((uint32_t)b[34 * (2 * w + q) + 1] << 8)) << (16 * q);
        }
    } else {
        if (wi < 512) {                              // bit-sliced e2m1 codes
            unit(wi, P, g, t, a, h);
            const uint8_t* b = blk_of(g + 8 * h);
            if (b)
                for (int u = 0; u < 2; ++u)
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t c = raw_code<FMT>(b, 16 * (4 * P + 2 * a + u) + 4 * t + i);
                        const int v = 2 * u + (i & 1), j = i >> 1;
                        out |= ((c & 7u) << (9 - 3 * v + 16 * j)) | ((c >> 3) << ((v == 0 ? 15 : 11 + v) + 16 * j));
                    }
        } else {                                     // 16 scale bytes per row: byte s = scale byte (s & 3) of 64-block s >> 2
            const int r = (wi - 512) >> 2, w = (wi - 512) & 3;
            const uint8_t* b = blk_of(r);
            if (b)
                for (int i = 0; i < 4; ++i) out |= (uint32_t)b[36 * w + i] << (8 * i);
        }
    }
    reinterpret_cast<uint32_t*>(t16)[gw] = out;
}

// one thread per stored byte of a 256-input block
template <int FMT>
__global__ void t16_to_raw_kernel(const uint8_t* __restrict__ t16, int64_t n, int64_t nb, uint8_t* __restrict__ raw, int64_t total_bytes) {
    constexpr int TB = kyb_tile_bytes(FMT);
    constexpr int RB = kyb_raw_kblock_bytes(FMT);
    const int64_t gb = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gb >= total_bytes) return;
    const int64_t blk = gb / RB;
    const int o = (int)(gb % RB);
    const int64_t row = blk / nb, kb = blk % nb;
    const uint8_t* tile = t16 + ((row >> 4) * nb + kb) * TB;
    const int r = (int)(row & 15);
    uint32_t out = 0;
    if (FMT == KYB_FMT_Q4_K) {
        if (o < 16) out = tile[2048 + r * 16 + o];
        else {
            const int G = (o - 16) >> 5, l = (o - 16) & 31;
            out = tile_code<FMT>(tile, r, 64 * G + l) | (tile_code<FMT>(tile, r, 64 * G + 32 + l) << 4);
        }
    } else if (FMT == KYB_FMT_Q6_K) {
        if (o < 128) {
            const int H = o >> 6, run = (o >> 5) & 1, l = o & 31;
            out = (tile_code<FMT>(tile, r, 128 * H + 32 * run + l) & 15u) | ((tile_code<FMT>(tile, r, 128 * H + 32 * (run + 2) + l) & 15u) << 4);
        } else if (o < 192) {
            const int H = (o - 128) >> 5, l = (o - 128) & 31;
            for (int i = 0; i < 4; ++i) out |= (tile_code<FMT>(tile, r, 128 * H + 32 * i + l) >> 4) << (2 * i);
        } else if (o < 208) out = tile[3072 + r * 16 + (o - 192)];
        else out = tile[3328 + r * 2 + (o - 208)];
    } else if (FMT == KYB_FMT_Q3_K) {
        if (o < 32) {
            for (int i = 0; i < 8; ++i) out |= (tile_code<FMT>(tile, r, 128 * (i >> 2) + 32 * (i & 3) + o) >> 2) << i;
        } else if (o < 96) {
            const int H = (o - 32) >> 5, l = (o - 32) & 31;
            for (int j = 0; j < 4; ++j) out |= (tile_code<FMT>(tile, r, 128 * H + 32 * j + l) & 3u) << (2 * j);
        } else if (o < 108) out = tile[1536 + r * 12 + (o - 96)];
        else out = tile[1728 + r * 2 + (o - 108)];
    } else if (FMT == KYB_FMT_Q5_K) {
        if (o < 16) out = tile[2560 + r * 16 + o];
        else if (o < 48) {
            for (int i = 0; i < 8; ++i) out |= (tile_code<FMT>(tile, r, 32 * i + (o - 16)) >> 4) << i;
        } else {
            const int G = (o - 48) >> 5, l = (o - 48) & 31;
            out = (tile_code<FMT>(tile, r, 64 * G + l) & 15u) | ((tile_code<FMT>(tile, r, 64 * G + 32 + l) & 15u) << 4);
        }
    } else if (FMT == KYB_FMT_IQ4_XS) {
        if (o < 8) out = tile[2048 + r * 8 + o];
        else {
            const int ib = (o - 8) >> 4, j = (o - 8) & 15;
            out = tile_code<FMT>(tile, r, 32 * ib + j) | (tile_code<FMT>(tile, r, 32 * ib + 16 + j) << 4);
        }
    } else if (FMT == KYB_FMT_Q2_K) {
        if (o < 16) out = tile[1024 + r * 16 + o];
        else if (o < 80) {
            const int H = (o - 16) >> 5, l = (o - 16) & 31;
            for (int j = 0; j < 4; ++j) out |= tile_code<FMT>(tile, r, 128 * H + 32 * j + l) << (2 * j);
        } else out = tile[1280 + r * 4 + (o - 80)];
    } else if (FMT == KYB_FMT_Q8_0) {
        const int B = o / 34, p = o % 34;
        out = p < 2 ? tile[4096 + r * 16 + 2 * B + p] : tile_code<FMT>(tile, r, 32 * B + p - 2);
    } else {
        const int B = o / 36, p = o % 36;
        if (p < 4) out = tile[2048 + r * 16 + 4 * B + p];
        else {
            const int u = (p - 4) >> 3, l = (p - 4) & 7;
            const int e = 64 * B + 16 * u + l;
            out = tile_code<FMT>(tile, r, e) | (tile_code<FMT>(tile, r, e + 8) << 4);
        }
    }
    raw[gb] = (uint8_t)out;
}

}  // namespace kyb

static int check_fmt_shape(int fmt, int64_t n, int64_t k) {
    KYB_REQUIRE(fmt >= 0 && fmt < KYB_FMT_COUNT, "unknown weight format %d", fmt);
    KYB_REQUIRE(n > 0 && k > 0 && k % 256 == 0, "n=%lld k=%lld: n must be positive and k a positive multiple of 256", (long long)n, (long long)k);
    return KYB_OK;
}

extern "C" int kyb_repack_raw_to_t16(int fmt, const void* raw, int64_t n, int64_t k, void* t16, void* stream) {
    if (int s = check_fmt_shape(fmt, n, k)) return s;
    KYB_REQUIRE(raw && t16, "null pointer");
    KYB_REQUIRE(((uintptr_t)t16 & 15) == 0, "t16 must be 16-byte aligned");
    const int64_t nb = k / 256, words = (int64_t)(kyb_t16_nbytes(fmt, n, k) / 4);
    const int threads = 256;
    const unsigned blocks = (unsigned)((words + threads - 1) / threads);
    cudaStream_t st = (cudaStream_t)stream;
    const uint8_t* r = (const uint8_t*)raw;
    uint8_t* o = (uint8_t*)t16;
    switch (fmt) {
        case KYB_FMT_Q4_K: kyb::raw_to_t16_kernel<KYB_FMT_Q4_K><<<blocks, threads, 0, st>>>(r, n, nb, o, words); break;
        case KYB_FMT_Q6_K: kyb::raw_to_t16_kernel<KYB_FMT_Q6_K><<<blocks, threads, 0, st>>>(r, n, nb, o, words); break;
        case KYB_FMT_Q3_K: kyb::raw_to_t16_kernel<KYB_FMT_Q3_K><<<blocks, threads, 0, st>>>(r, n, nb, o, words); break;
        case KYB_FMT_Q5_K: kyb::raw_to_t16_kernel<KYB_FMT_Q5_K><<<blocks, threads, 0, st>>>(r, n, nb, o, words); break;
        case KYB_FMT_Q8_0: kyb::raw_to_t16_kernel<KYB_FMT_Q8_0><<<blocks, threads, 0, st>>>(r, n, nb, o, words); break;
        case KYB_FMT_Q2_K: kyb::raw_to_t16_kernel<KYB_FMT_Q2_K><<<blocks, threads, 0, st>>>(r, n, nb, o, words); break;
        case KYB_FMT_IQ4_XS: kyb::raw_to_t16_kernel<KYB_FMT_IQ4_XS><<<blocks, threads, 0, st>>>(r, n, nb, o, words); break;
        default: kyb::raw_to_t16_kernel<KYB_FMT_NVFP4><<<blocks, threads, 0, st>>>(r, n, nb, o, words); break;
    }
    return kyb_launch_check("raw_to_t16");
}

extern "C" int kyb_repack_t16_to_raw(int fmt, const void* t16, int64_t n, int64_t k, void* raw, void* stream) {
    if (int s = check_fmt_shape(fmt, n, k)) return s;
    KYB_REQUIRE(raw && t16, "null pointer");
    KYB_REQUIRE(((uintptr_t)t16 & 15) == 0, "t16 must be 16-byte aligned");
    const int64_t nb = k / 256, bytes = n * (int64_t)kyb_raw_row_bytes(fmt, k);
    const int threads = 256;
    const unsigned blocks = (unsigned)((bytes + threads - 1) / threads);
    cudaStream_t st = (cudaStream_t)stream;
    const uint8_t* t = (const uint8_t*)t16;
    uint8_t* o = (uint8_t*)raw;
    switch (fmt) {
        case KYB_FMT_Q4_K: kyb::t16_to_raw_kernel<KYB_FMT_Q4_K><<<blocks, threads, 0, st>>>(t, n, nb, o, bytes); break;
        case KYB_FMT_Q6_K: kyb::t16_to_raw_kernel<KYB_FMT_Q6_K><<<blocks, threads, 0, st>>>(t, n, nb, o, bytes); break;
        case KYB_FMT_Q3_K: kyb::t16_to_raw_kernel<KYB_FMT_Q3_K><<<blocks, threads, 0, st>>>(t, n, nb, o, bytes); break;
        case KYB_FMT_Q5_K: kyb::t16_to_raw_kernel<KYB_FMT_Q5_K><<<blocks, threads, 0, st>>>(t, n, nb, o, bytes); break;
        case KYB_FMT_Q8_0: kyb::t16_to_raw_kernel<KYB_FMT_Q8_0><<<blocks, threads, 0, st>>>(t, n, nb, o, bytes); break;
        case KYB_FMT_Q2_K: kyb::t16_to_raw_kernel<KYB_FMT_Q2_K><<<blocks, threads, 0, st>>>(t, n, nb, o, bytes); break;
        case KYB_FMT_IQ4_XS: kyb::t16_to_raw_kernel<KYB_FMT_IQ4_XS><<<blocks, threads, 0, st>>>(t, n, nb, o, bytes); break;
        default: kyb::t16_to_raw_kernel<KYB_FMT_NVFP4><<<blocks, threads, 0, st>>>(t, n, nb, o, bytes); break;
    }
    return kyb_launch_check("t16_to_raw");
}
