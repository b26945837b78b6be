// T16 -> row-major [n, k] float32 / float16. One warp per tile; lane (g, t) writes 4 consecutive weights of rows g and
// g + 8 for each of the 16 MMA slices, so a row's 64-byte run of a slice is written by four adjacent lanes.
#include "t16_decode.cuh"

namespace kyb {

template <int FMT, typename OUT>
__global__ void dequant_t16_kernel(const uint8_t* __restrict__ t16, int64_t n, int64_t nb, int64_t rt0, int64_t ntiles, float gscale,
                                   OUT* __restrict__ out, int64_t ld) {
    constexpr int TB = kyb_tile_bytes(FMT);
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (warp >= ntiles) return;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int64_t rt = rt0 + warp / nb, kb = warp % nb;
    const uint8_t* tile = t16 + (rt * nb + kb) * TB;
#pragma unroll 1
    for (int h = 0; h < 2; ++h) {
        const int64_t row = rt * 16 + g + 8 * h;
        if (row >= n) continue;
        OUT* dst = out + (row - rt0 * 16) * ld + kb * 256 + 4 * t;
#pragma unroll 4
        for (int s = 0; s < 16; ++s) {
            float w[4];
            TileDecode<FMT>::row4(tile, g, t, h, s, gscale, w);
            if constexpr (sizeof(OUT) == 4) {
                *reinterpret_cast<float4*>(dst + 16 * s) = make_float4(w[0], w[1], w[2], w[3]);
            } else {
                __half2 lo = sat_half2(w[0], w[1]), hi = sat_half2(w[2], w[3]);
                uint2 v;
                v.x = *reinterpret_cast<uint32_t*>(&lo);
                v.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(dst + 16 * s) = v;
            }
        }
    }
}

// Gathered rows: out[i] = decoded row rows[i] (token-embedding lookup in the stored blocks, kyojin_mlx/foreign_linear.py:1170-1199). One warp per
// (requested row, 256-input block); lane L decodes the two 4-weight runs (t, s) = (L & 3, L >> 2) and (L & 3, 8 + (L >> 2)) of that row.
template <int FMT, typename OUT>
__global__ void dequant_rows_kernel(const uint8_t* __restrict__ t16, int64_t n, int64_t nb, const int32_t* __restrict__ rows, int64_t nrows, float gscale,
                                    OUT* __restrict__ out, int64_t ld) {
    constexpr int TB = kyb_tile_bytes(FMT);
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (warp >= nrows * nb) return;
    const int lane = threadIdx.x & 31;
    const int64_t i = warp / nb, kb = warp % nb;
    int64_t row = rows[i];
    if (row < 0 || row >= n) row = 0;                                    // the host contract is 0 <= id < n; a bad id never reads outside the table
    const uint8_t* tile = t16 + ((row >> 4) * nb + kb) * TB;
    const int g = (int)(row & 7), h = (int)((row >> 3) & 1), t = lane & 3;
    OUT* dst = out + i * ld + kb * 256 + 4 * t;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int s = (lane >> 2) + 8 * half;
        float w[4];
        TileDecode<FMT>::row4(tile, g, t, h, s, gscale, w);
        if constexpr (sizeof(OUT) == 4) {
            *reinterpret_cast<float4*>(dst + 16 * s) = make_float4(w[0], w[1], w[2], w[3]);
        } else {
            __half2 lo = sat_half2(w[0], w[1]), hi = sat_half2(w[2], w[3]);
            uint2 v;
            v.x = *reinterpret_cast<uint32_t*>(&lo);
            v.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(dst + 16 * s) = v;
        }
    }
}

}  // namespace kyb

template <int FMT>
static void launch_dequant(const uint8_t* t16, int64_t n, int64_t nb, int64_t rt0, int64_t ntiles, float gscale, int dt, void* out, int64_t ld, cudaStream_t st) {
    const int threads = 256;
    const unsigned blocks = (unsigned)((ntiles * 32 + threads - 1) / threads);
    if (dt == KYB_DT_F32) kyb::dequant_t16_kernel<FMT, float><<<blocks, threads, 0, st>>>(t16, n, nb, rt0, ntiles, gscale, (float*)out, ld);
    else kyb::dequant_t16_kernel<FMT, __half><<<blocks, threads, 0, st>>>(t16, n, nb, rt0, ntiles, gscale, (__half*)out, ld);
}

extern "C" int kyb_dequant_t16(int fmt, const void* t16, int64_t n, int64_t k, int64_t row0, int64_t nrows, float gscale, int out_dtype, void* out,
                               int64_t ld, void* stream) {
    KYB_REQUIRE(fmt >= 0 && fmt < KYB_FMT_COUNT, "unknown weight format %d", fmt);
    KYB_REQUIRE(n > 0 && k > 0 && k % 256 == 0, "n=%lld k=%lld: k must be a positive multiple of 256", (long long)n, (long long)k);
    KYB_REQUIRE(t16 && out, "null pointer");
    KYB_REQUIRE(out_dtype == KYB_DT_F32 || out_dtype == KYB_DT_F16, "out_dtype %d is neither KYB_DT_F32 nor KYB_DT_F16", out_dtype);
    KYB_REQUIRE(row0 >= 0 && row0 % 16 == 0 && nrows > 0 && row0 + nrows <= n, "rows [%lld, %lld) outside [0, %lld) or row0 %% 16 != 0", (long long)row0,
                (long long)(row0 + nrows), (long long)n);
    KYB_REQUIRE(ld >= k && ld % 4 == 0, "ld=%lld must be >= k and a multiple of 4", (long long)ld);
    KYB_REQUIRE(((uintptr_t)t16 & 15) == 0 && ((uintptr_t)out & 15) == 0, "t16 and out must be 16-byte aligned");
    const int64_t nb = k / 256, rt0 = row0 / 16, ntiles = ((nrows + 15) / 16) * nb;
    const int64_t nlim = row0 + nrows;          // rows past the requested range are not written
    cudaStream_t st = (cudaStream_t)stream;
    const uint8_t* t = (const uint8_t*)t16;
    switch (fmt) {
        case KYB_FMT_Q4_K: launch_dequant<KYB_FMT_Q4_K>(t, nlim, nb, rt0, ntiles, gscale, out_dtype, out, ld, st); break;
        case KYB_FMT_Q6_K: launch_dequant<KYB_FMT_Q6_K>(t, nlim, nb, rt0, ntiles, gscale, out_dtype, out, ld, st); break;
        case KYB_FMT_Q3_K: launch_dequant<KYB_FMT_Q3_K>(t, nlim, nb, rt0, ntiles, gscale, out_dtype, out, ld, st); break;
        case KYB_FMT_Q5_K: launch_dequant<KYB_FMT_Q5_K>(t, nlim, nb, rt0, ntiles, gscale, out_dtype, out, ld, st); break;
        case KYB_FMT_Q8_0: launch_dequant<KYB_FMT_Q8_0>(t, nlim, nb, rt0, ntiles, gscale, out_dtype, out, ld, st); break;
        case KYB_FMT_Q2_K: launch_dequant<KYB_FMT_Q2_K>(t, nlim, nb, rt0, ntiles, gscale, out_dtype, out, ld, st); break;
        case KYB_FMT_IQ4_XS: launch_dequant<KYB_FMT_IQ4_XS>(t, nlim, nb, rt0, ntiles, gscale, out_dtype, out, ld, st); break;
        default: launch_dequant<KYB_FMT_NVFP4>(t, nlim, nb, rt0, ntiles, gscale, out_dtype, out, ld, st); break;
    }
    return kyb_launch_check("dequant_t16");
}

template <int FMT>
static void launch_dequant_rows(const uint8_t* t16, int64_t n, int64_t nb, const int32_t* rows, int64_t nrows, float gscale, int dt, void* out, int64_t ld, cudaStream_t st) {
    const int threads = 256;
    const unsigned blocks = (unsigned)((nrows * nb * 32 + threads - 1) / threads);
    if (dt == KYB_DT_F32) kyb::dequant_rows_kernel<FMT, float><<<blocks, threads, 0, st>>>(t16, n, nb, rows, nrows, gscale, (float*)out, ld);
    else kyb::dequant_rows_kernel<FMT, __half><<<blocks, threads, 0, st>>>(t16, n, nb, rows, nrows, gscale, (__half*)out, ld);
}

extern "C" int kyb_dequant_rows_t16(int fmt, const void* t16, int64_t n, int64_t k, const void* rows, int64_t nrows, float gscale, int out_dtype, void* out, int64_t ld,
                                    void* stream) {
    KYB_REQUIRE(fmt >= 0 && fmt < KYB_FMT_COUNT, "unknown weight format %d", fmt);
    KYB_REQUIRE(n > 0 && k > 0 && k % 256 == 0, "n=%lld k=%lld: k must be a positive multiple of 256", (long long)n, (long long)k);
    KYB_REQUIRE(t16 && rows && out, "null pointer");
    KYB_REQUIRE(out_dtype == KYB_DT_F32 || out_dtype == KYB_DT_F16, "out_dtype %d is neither KYB_DT_F32 nor KYB_DT_F16", out_dtype);
    KYB_REQUIRE(nrows > 0 && nrows * (k / 256) < (1ll << 31), "nrows=%lld out of range", (long long)nrows);
    KYB_REQUIRE(ld >= k && ld % 4 == 0, "ld=%lld must be >= k and a multiple of 4", (long long)ld);
    KYB_REQUIRE(((uintptr_t)t16 & 15) == 0 && ((uintptr_t)out & 15) == 0, "t16 and out must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const uint8_t* t = (const uint8_t*)t16;
    const int32_t* r = (const int32_t*)rows;
    const int64_t nb = k / 256;
    switch (fmt) {
        case KYB_FMT_Q4_K: launch_dequant_rows<KYB_FMT_Q4_K>(t, n, nb, r, nrows, gscale, out_dtype, out, ld, st); break;
        case KYB_FMT_Q6_K: launch_dequant_rows<KYB_FMT_Q6_K>(t, n, nb, r, nrows, gscale, out_dtype, out, ld, st); break;
        case KYB_FMT_Q3_K: launch_dequant_rows<KYB_FMT_Q3_K>(t, n, nb, r, nrows, gscale, out_dtype, out, ld, st); break;
        case KYB_FMT_Q5_K: launch_dequant_rows<KYB_FMT_Q5_K>(t, n, nb, r, nrows, gscale, out_dtype, out, ld, st); break;
        case KYB_FMT_Q8_0: launch_dequant_rows<KYB_FMT_Q8_0>(t, n, nb, r, nrows, gscale, out_dtype, out, ld, st); break;
        case KYB_FMT_Q2_K: launch_dequant_rows<KYB_FMT_Q2_K>(t, n, nb, r, nrows, gscale, out_dtype, out, ld, st); break;
        case KYB_FMT_IQ4_XS: launch_dequant_rows<KYB_FMT_IQ4_XS>(t, n, nb, r, nrows, gscale, out_dtype, out, ld, st); break;
        default: launch_dequant_rows<KYB_FMT_NVFP4>(t, n, nb, r, nrows, gscale, out_dtype, out, ld, st); break;
    }
    return kyb_launch_check("dequant_rows_t16");
}
