// NVFP4 (e2m1 values, one e4m3 scale per 16 inputs) on the block-scaled tensor-core path of sm_100a.
//   nvfp4_quant_rows   activations bf16/fp16 -> packed e2m1 codes + e4m3 block scales, the rule of kyojin_mlx/fp4pack.py:30-48 `pack(x, 16, e4m3_scale=True)`
//   nvfp4_unpack_rows  inverse (fp4pack.py:51-63 `unpack`)
//   sf_swizzle         plain scale bytes [rows, k/16] -> the 128-row x 4-scale chunks tcgen05 reads (and back): lossless re-layout
//   gemm_nvfp4         D = sat(gscale * A B^T), A, B packed e2m1 [rows, k/2] K-major with block scales, tcgen05.mma kind::mxf4nvf4 block16, fp32 accumulate in TMEM
//
// Scale-factor chunk layout ("SF512"): rows are cut in blocks of 128, k in blocks of 64 (= 4 scales); chunk (rb, kb) holds 512 bytes at ((rb * k/64) + kb) * 512,
// byte (r % 32) * 16 + (r / 32) * 4 + c = scale c of row r of the block. One chunk is what `tcgen05.cp 32x128b.warpx4` moves into 4 tensor-memory columns.
#include <cuda_bf16.h>

#include <cstring>
#include <cuda_fp8.h>

#include <mutex>

#include "tc_common.cuh"

namespace kyb {

__device__ __forceinline__ float e4m3_to_float(uint32_t b) {      // unsigned e4m3 magnitude, exact (see e4m3_unsigned in t16_decode.cuh); 0x7F -> 0
    b &= 127u;
    const float v = __uint_as_float(b << 20) * 1.329227995784916e36f;
    return b == 127u ? 0.0f : v;
}

__device__ __forceinline__ size_t sf512_offset(int64_t row, int64_t s, int64_t kblocks64) {     // s = scale index along k (k / 16)
    const int64_t rb = row >> 7, r = row & 127, kb = s >> 2, c = s & 3;
    return (size_t)((rb * kblocks64 + kb) * 512 + (r & 31) * 16 + (r >> 5) * 4 + c);
}

// One thread per block of 16 inputs, four lanes per 4-byte group of the scale layouts. Per block: amax = max(|x|, 6 * 2^-9); scale byte = e4m3_rn(amax / 6) (true
// fp32 divide); v = clip(x / scale, -6, 6); code = #(|v| > .25, 1.25, 2.5, 5) + #(|v| >= .75, 1.75, 3.5) (round to nearest even onto e2m1), sign bit 3 for v < 0;
// two codes per byte, low first (kyojin_mlx/fp4pack.py:30-48).
// The quotient itself is never formed: for 16-bit inputs fl(|x| / s) > t holds exactly when |x| > t s (t s is exact in fp32, and a 16-bit |x| above t s exceeds it
// by at least 2^-11 relative, far more than half an fp32 ulp, so the correctly rounded quotient cannot land on t), likewise for >=; the clip at 6 only touches
// values that already passed the last threshold. The sign of the code is the sign of x with +-0 and underflowed quotients mapped as the division would: x / s is
// negative exactly when x < 0 (s > 0, and a non-zero 16-bit x over s <= 448 does not underflow to zero in fp32).
// Packed 16-bit arithmetic of the quantiser: two inputs per instruction in their own type. Every threshold t s has at most 7 significant bits, so it is exact in
// fp16 and in bf16, and the comparisons |x| > t s / |x| >= t s give the same truth values as in fp32.
template <typename T>
struct Pk;
template <>
struct Pk<__half> {
    using V = __half2;
    static __device__ __forceinline__ V splat(float f) { return __float2half2_rn(f); }
    static __device__ __forceinline__ float hi_lo_max(V m) { return fmaxf(__low2float(m), __high2float(m)); }
    static constexpr uint32_t MAGIC = 0x64006400u;                        // 1024 + code is exact: the code sits in the low mantissa bits
};
template <>
struct Pk<__nv_bfloat16> {
    using V = __nv_bfloat162;
    static __device__ __forceinline__ V splat(float f) { return __float2bfloat162_rn(f); }
    static __device__ __forceinline__ float hi_lo_max(V m) { return fmaxf(__low2float(m), __high2float(m)); }
    static constexpr uint32_t MAGIC = 0x43004300u;                        // 128 + code (code < 16) is exact in bf16
};

template <typename T>
__global__ void __launch_bounds__(256) nvfp4_quant_rows_kernel(const T* __restrict__ x, int64_t ldx, int64_t rows, int64_t k, uint8_t* __restrict__ codes,
                                                               uint8_t* __restrict__ sf_plain, uint8_t* __restrict__ sf_swz) {
    // one thread per block of 16 inputs (two 16-byte loads; a warp reads 1 KB of a row contiguously); the four lanes of a 64-input group combine their scale bytes
    // with shuffles and one of them writes the 4-byte group of both scale layouts
    using V = typename Pk<T>::V;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nblk = k >> 4, total = rows * nblk;
    const bool live = i < total;
    const int64_t ii = live ? i : total - 1;                               // lanes past the end repeat the last block (no stores) so that the shuffles stay full-warp
    const int64_t row = ii / nblk, b = ii % nblk;
    const uint4* xp = reinterpret_cast<const uint4*>(x + row * ldx + b * 16);
    const uint4 r0 = __ldg(xp), r1 = __ldg(xp + 1);
    const uint32_t w[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
    V a[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t m = w[j] & 0x7FFF7FFFu;
        a[j] = *reinterpret_cast<const V*>(&m);
    }
    V mx = a[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) mx = __hmax2(mx, a[j]);
    const float amax = fmaxf(6.0f * 0.001953125f, Pk<T>::hi_lo_max(mx));
    const uint32_t s8 = (uint32_t)__nv_cvt_float_to_fp8(__fdiv_rn(amax, 6.0f), __NV_SATFINITE, __NV_E4M3) & 255u;
    const float scale = e4m3_to_float(s8);
    const V t0 = Pk<T>::splat(0.25f * scale), t1 = Pk<T>::splat(0.75f * scale), t2 = Pk<T>::splat(1.25f * scale), t3 = Pk<T>::splat(1.75f * scale),
            t4 = Pk<T>::splat(2.5f * scale), t5 = Pk<T>::splat(3.5f * scale), t6 = Pk<T>::splat(5.0f * scale);
    const V zero = Pk<T>::splat(0.0f), eight = Pk<T>::splat(8.0f);
    const uint32_t magic_bits = Pk<T>::MAGIC;
    const V magic = *reinterpret_cast<const V*>(&magic_bits);
    uint32_t pk[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        // number of thresholds passed = the e2m1 magnitude code (each comparison yields 1.0 or 0.0 per half)
        V c = __hadd2(__hadd2(__hadd2(__hgt2(a[j], t0), __hge2(a[j], t1)), __hadd2(__hgt2(a[j], t2), __hge2(a[j], t3))),
                      __hadd2(__hadd2(__hgt2(a[j], t4), __hge2(a[j], t5)), __hgt2(a[j], t6)));
        c = __hfma2(__hlt2(*reinterpret_cast<const V*>(&w[j]), zero), eight, c);          // sign bit 3 for x < 0 (not for -0)
        c = __hadd2(c, magic);
        const uint32_t u = *reinterpret_cast<const uint32_t*>(&c) & 0x000F000Fu;
        pk[j >> 2] |= ((u | (u >> 12)) & 0xFFu) << (8 * (j & 3));
    }
    if (live) *reinterpret_cast<uint2*>(codes + row * (k >> 1) + b * 8) = make_uint2(pk[0], pk[1]);
    // scale bytes of the 64-input group (k % 64 == 0, so a group never straddles two rows and its four lanes sit in one warp)
    const int lane = threadIdx.x & 31;
    uint32_t word = s8 << (8 * (lane & 3));
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    word |= __shfl_xor_sync(0xffffffffu, word, 2);
    if (live && (lane & 3) == 0) {
        if (sf_plain) *reinterpret_cast<uint32_t*>(sf_plain + row * nblk + b) = word;
        if (sf_swz) *reinterpret_cast<uint32_t*>(sf_swz + sf512_offset(row, b, k >> 6)) = word;
    }
}

// General form (any k % 16 == 0, any alignment): one thread per block of 16 inputs, the quotient formed with a true divide. amax = max(|x|, 6 * 2^-9); scale byte = e4m3_rn(amax / 6); v = clip(x / scale, -6, 6);
// code = #(|v| > .25, 1.25, 2.5, 5) + #(|v| >= .75, 1.75, 3.5) (round to nearest even onto e2m1), sign bit 3 for v < 0; two codes per byte, low first.
template <typename T>
__global__ void nvfp4_quant_rows16_kernel(const T* __restrict__ x, int64_t ldx, int64_t rows, int64_t k, uint8_t* __restrict__ codes, uint8_t* __restrict__ sf_plain,
                                        uint8_t* __restrict__ sf_swz) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nblk = k >> 4;
    if (i >= rows * nblk) return;
    const int64_t row = i / nblk, b = i % nblk;
    const T* xp = x + row * ldx + b * 16;
    float v[16];
    float amax = 6.0f * 0.001953125f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        v[j] = (float)xp[j];
        amax = fmaxf(amax, fabsf(v[j]));
    }
    const uint8_t s8 = (uint8_t)__nv_cvt_float_to_fp8(__fdiv_rn(amax, 6.0f), __NV_SATFINITE, __NV_E4M3);
    const float scale = e4m3_to_float(s8);
    uint32_t packed[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const float q = fminf(fmaxf(__fdiv_rn(v[j], scale), -6.0f), 6.0f);
        const float mag = fabsf(q);
        const uint32_t code = (uint32_t)(mag > 0.25f) + (uint32_t)(mag > 1.25f) + (uint32_t)(mag > 2.5f) + (uint32_t)(mag > 5.0f) + (uint32_t)(mag >= 0.75f) +
                              (uint32_t)(mag >= 1.75f) + (uint32_t)(mag >= 3.5f);
        packed[j >> 3] |= (code | (q < 0.0f ? 8u : 0u)) << (4 * (j & 7));
    }
    *reinterpret_cast<uint2*>(codes + row * (k >> 1) + b * 8) = make_uint2(packed[0], packed[1]);
    if (sf_plain) sf_plain[row * nblk + b] = s8;
    if (sf_swz) sf_swz[sf512_offset(row, b, k >> 6)] = s8;
}

template <typename T>
__global__ void nvfp4_unpack_rows_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ sf_plain, int64_t rows, int64_t k, T* __restrict__ out, int64_t ldo) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nblk = k >> 4;
    if (i >= rows * nblk) return;
    const int64_t row = i / nblk, b = i % nblk;
    const uint2 pk = *reinterpret_cast<const uint2*>(codes + row * (k >> 1) + b * 8);
    const float scale = e4m3_to_float(sf_plain[row * nblk + b]);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const uint32_t c = ((j < 8 ? pk.x : pk.y) >> (4 * (j & 7))) & 15u;
        const uint32_t hb = ((c & 8u) << 12) | ((c & 7u) << 9);                       // e2m1 as fp16 bits = value * 2^-14
        out[row * ldo + b * 16 + j] = (T)(half_bits_to_float(hb) * 16384.0f * scale);
    }
}

// ---- the block-32 form with a power-of-two scale (one exponent byte per 32 values; the reference's second branch of kyojin_mlx/fp4pack.py:30-63).
// One thread per block: scale = 2^e with e = ceil(log2(max(amax, 6 * 2^-126) / 6)), stored as e + 127; values are divided by the scale exactly (a power of two),
// clipped to +-6 and take the e2m1 code by the same thresholds as the block-16 form. e is the mathematical ceiling of the logarithm of the float32 quotient,
// read from its exponent and mantissa bits (no library logarithm in the way).
template <typename T>
__global__ void fp4_quant_block32_kernel(const T* __restrict__ x, int64_t ldx, int64_t rows, int64_t k, uint8_t* __restrict__ codes, uint8_t* __restrict__ sbytes) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nblk = k >> 5;
    if (i >= rows * nblk) return;
    const int64_t row = i / nblk, b = i % nblk;
    const T* xp = x + row * ldx + b * 32;
    float v[32], amax = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = (float)xp[j], amax = fmaxf(amax, fabsf(v[j]));
    const float q = fmaxf(amax, 6.0f * 1.1754943508222875e-38f) / 6.0f;                 // >= 2^-126: a normal float32
    const uint32_t qb = __float_as_uint(q);
    const int e = (int)(qb >> 23) - 127 + ((qb & 0x7FFFFFu) ? 1 : 0);                    // ceil(log2 q)
    const float inv = __uint_as_float((uint32_t)(127 - e) << 23);                          // 2^-e (e in [-126, 13] for 16-bit inputs)
    sbytes[row * nblk + b] = (uint8_t)(e + 127);
    uint8_t* cp = codes + row * (k >> 1) + b * 16;
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
        uint32_t pair = 0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float w = fminf(fmaxf(v[j + h] * inv, -6.0f), 6.0f), mag = fabsf(w);
            const uint32_t c = (mag > 0.25f) + (mag > 1.25f) + (mag > 2.5f) + (mag > 5.0f) + (mag >= 0.75f) + (mag >= 1.75f) + (mag >= 3.5f);
            pair |= (c | (w < 0.f ? 8u : 0u)) << (4 * h);
        }
        cp[j >> 1] = (uint8_t)pair;
    }
}

template <typename T>
__global__ void fp4_unpack_block32_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ sbytes, int64_t rows, int64_t k, T* __restrict__ out, int64_t ldo) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nblk = k >> 5;
    if (i >= rows * nblk) return;
    const int64_t row = i / nblk, b = i % nblk;
    const uint4 pk = *reinterpret_cast<const uint4*>(codes + row * (k >> 1) + b * 16);
    const uint32_t words[4] = {pk.x, pk.y, pk.z, pk.w};
    const float scale = exp2f((float)sbytes[row * nblk + b] - 127.0f);                  // exact for integer arguments
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const uint32_t c = (words[j >> 3] >> (4 * (j & 7))) & 15u;
        const uint32_t hb = ((c & 8u) << 12) | ((c & 7u) << 9);                       // e2m1 as fp16 bits = value * 2^-14
        out[row * ldo + b * 32 + j] = (T)(half_bits_to_float(hb) * 16384.0f * scale);
    }
}

// plain [rows, k/16] <-> SF512 (rows padded to 128 with zero scales); sanitize: sign bit dropped, NaN code 0x7F -> 0 (the reference's decode rule)
__global__ void sf_swizzle_kernel(const uint8_t* __restrict__ plain, int64_t rows, int64_t k, uint8_t* __restrict__ swz, int to_swizzled) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nblk = k >> 4, rows_pad = (rows + 127) & ~(int64_t)127;
    if (i >= rows_pad * nblk) return;
    const int64_t row = i / nblk, s = i % nblk;
    const size_t o = sf512_offset(row, s, k >> 6);
    if (to_swizzled) {
        uint8_t v = row < rows ? (uint8_t)(plain[row * nblk + s] & 127u) : (uint8_t)0;
        swz[o] = v == 127 ? (uint8_t)0 : v;
    } else if (row < rows) {
        const_cast<uint8_t*>(plain)[row * nblk + s] = swz[o];
    }
}

// ------------------------------------------------------------------------------------------------ block-scaled GEMM
constexpr int NV_BM = 128, NV_BN = 256, NV_BK = 256, NV_THREADS = 192, NV_STAGES = 4;
constexpr uint32_t NV_A_BYTES = NV_BM * NV_BK / 2, NV_B_BYTES = NV_BN * NV_BK / 2, NV_SFA_BYTES = 4 * 512, NV_SFB_BYTES = 2 * 4 * 512;
constexpr uint32_t NV_STAGE_BYTES = NV_A_BYTES + NV_B_BYTES + NV_SFA_BYTES + NV_SFB_BYTES;     // 16 K + 32 K + 2 K + 4 K

struct NvGemmParams {
    const uint8_t* sfa;      // SF512 of A [m_pad / 128][k / 64][512]
    const uint8_t* sfb;      // SF512 of B
    __half* d[8];            // output matrix on every receiving rank (one entry without sharding), already offset to this rank's first column
    int nout;
    int tma_out, col0;       // the epilogue stores through the tensor maps (tiled bulk stores) at column col0 + n0
    int wide, stages;        // 32 x 64 boxes (outputs that also go to other GPUs; one pipeline stage fewer to make room for the staging), ring depth
    int64_t ldd;
    int m, n, k;
    float gscale;
    int out_bf16;
    unsigned int* status;
};

// kind::mxf4nvf4 instruction descriptor: A = B = e2m1 (format 1 at [7,10) and [10,13)), scales ue4m3 (bit 23 = 0), K-major, N >> 3 at [17,23), M >> 4 at [24,29)
__host__ __device__ constexpr uint32_t umma_idesc_nvf4(int m, int n) { return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24); }

// shared-memory descriptor of one 512-byte scale chunk (32 rows of 16 bytes, no swizzle): 8-row groups 128 bytes apart
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}
__device__ __forceinline__ void tmem_cp_32x128b_x4(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma_nvf4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t tsfa, uint32_t tsfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(tsfa), "r"(tsfb), "r"(accumulate)
        : "memory");
}

// Persistent: CTA c works on tiles c, c + gridDim.x, ... (m tile fastest: the CTAs running together share a few weight tiles, the activation codes stay in L2). Tensor memory: accumulator 256 columns + scale columns; the producer runs ahead
// into the next tile while the epilogue drains the accumulator.
__global__ void __launch_bounds__(NV_THREADS, 1) gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                                                                   const __grid_constant__ KybOutMaps outs, const NvGemmParams p, const int tiles_n, const int num_tiles) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int STAGES = p.stages;
    const uint32_t stg0 = smem0 + STAGES * NV_STAGE_BYTES;                         // epilogue staging, 4 warps
    const uint32_t stg_bytes = p.wide ? 2 * KYB_STG_BYTES : KYB_STG_BYTES;
    const uint32_t bars = stg0 + 4 * stg_bytes;
    const uint32_t full0 = bars, empty0 = bars + 8 * STAGES, accf = bars + 16 * STAGES, acce = accf + 8, tmem_slot = acce + 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = p.k / NV_BK, k64 = p.k / 64;
    constexpr uint32_t TMEM_COLS = 512, COL_SFA = 256, COL_SFB = 272;       // accumulator [0, 256), scales of A [256, 272), of B [272, 304)

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init_a(full0 + 8 * s, 1), mbar_init_a(empty0 + 8 * s, 1);
        mbar_init_a(accf, 1);
        mbar_init_a(acce, 4);
        mbar_fence_init();
        prefetch_tmap(&tma_a);
        prefetch_tmap(&tma_b);
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = lds32(tmem_slot);
    bool failed = false;

    if (warp == 0) {
        if (elect_one()) {
            uint32_t parity = 1;
            int s = 0;
            for (int t = blockIdx.x; t < num_tiles && !failed; t += gridDim.x) {
                const int tiles_m = num_tiles / tiles_n, n0 = (t / tiles_m) * NV_BN, m0 = (t % tiles_m) * NV_BM;   // m fastest: CTAs running together share the weight rows
                for (int kb = 0; kb < kblocks && !failed; ++kb) {
                    if (!mbar_wait_fast(empty0 + 8 * s, parity)) failed = true;
                    const uint32_t a_dst = smem0 + s * NV_STAGE_BYTES, b_dst = a_dst + NV_A_BYTES, sfa_dst = b_dst + NV_B_BYTES, sfb_dst = sfa_dst + NV_SFA_BYTES;
                    const uint32_t bar = full0 + 8 * s;
                    mbar_expect_tx_a(bar, NV_STAGE_BYTES);
                    tma_load_2d(a_dst, &tma_a, kb * (NV_BK / 2), m0, bar);                 // coordinates in bytes along k (two codes per byte)
                    tma_load_2d(b_dst, &tma_b, kb * (NV_BK / 2), n0, bar);
                    const uint8_t* sa = p.sfa + ((size_t)(m0 >> 7) * k64 + (size_t)kb * 4) * 512;
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(sfa_dst), "l"(sa), "r"(NV_SFA_BYTES), "r"(bar) : "memory");
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint8_t* sb = p.sfb + ((size_t)((n0 >> 7) + h) * k64 + (size_t)kb * 4) * 512;
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(sfb_dst + h * 2048), "l"(sb), "r"(2048u), "r"(bar)
                                     : "memory");
                    }
                    if (++s == STAGES) s = 0, parity ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc = umma_idesc_nvf4(NV_BM, NV_BN);
            uint32_t parity = 0;
            int s = 0, it = 0;
            for (int t = blockIdx.x; t < num_tiles && !failed; t += gridDim.x, ++it) {
                if (!mbar_wait_fast(acce, ((uint32_t)it & 1u) ^ 1u)) failed = true;         // the epilogue has drained the accumulator
                tc_fence_after();
                for (int kb = 0; kb < kblocks && !failed; ++kb) {
                    if (!mbar_wait_fast(full0 + 8 * s, parity)) failed = true;
                    tc_fence_after();
                    const uint32_t a_src = smem0 + s * NV_STAGE_BYTES, b_src = a_src + NV_A_BYTES, sfa_src = b_src + NV_B_BYTES, sfb_src = sfa_src + NV_SFA_BYTES;
                    // scales of this stage into tensor memory: A 4 chunks (one per 64-wide k block), B 2 row blocks x 4 chunks; the copies and the MMAs of one
                    // thread execute in issue order, so the same columns are reused every stage
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        tmem_cp_32x128b_x4(tmem_base + COL_SFA + 4 * j, sf_desc(sfa_src + 512 * j));
                        tmem_cp_32x128b_x4(tmem_base + COL_SFB + 8 * j, sf_desc(sfb_src + 512 * j));
                        tmem_cp_32x128b_x4(tmem_base + COL_SFB + 8 * j + 4, sf_desc(sfb_src + 2048 + 512 * j));
                    }
                    const uint64_t adesc = umma_desc_sw128(a_src), bdesc = umma_desc_sw128(b_src);
#pragma unroll
                    for (int j = 0; j < 4; ++j)                                              // 64 e2m1 = 32 bytes along k inside the swizzle atom
                        umma_nvf4(tmem_base, adesc + 2 * j, bdesc + 2 * j, idesc, tmem_base + COL_SFA + 4 * j, tmem_base + COL_SFB + 8 * j, (kb | j) != 0);
                    umma_commit(empty0 + 8 * s);
                    if (++s == STAGES) s = 0, parity ^= 1u;
                }
                umma_commit(accf);
            }
        }
    } else {
        const int q = warp & 3;
        int it = 0;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
            const int tiles_m = num_tiles / tiles_n, n0 = (t / tiles_m) * NV_BN, m0 = (t % tiles_m) * NV_BM;   // m fastest: CTAs running together share the weight rows
            if (!mbar_wait_fast(accf, (uint32_t)it & 1u)) failed = true;
            tc_fence_after();
            if (p.tma_out) {
                // The accumulator is the only one, so the MMAs of the next tile wait for this read-out: all 8 steps of 32 columns are therefore first pulled into
                // registers as packed 16-bit pairs (the load of step c + 1 in flight while step c is converted), the accumulator is handed back, and only then
                // do the staged bulk stores run, under the next tile's MMAs.
                const uint32_t stg = stg0 + (uint32_t)q * stg_bytes;
                const int row0 = m0 + q * 32;
                const uint32_t tq = tmem_base + ((uint32_t)(q * 32) << 16);
                uint32_t w[NV_BN / 32][16];
                auto pack = [&](const uint32_t (&v)[32], uint32_t (&o)[16]) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float f0 = __uint_as_float(v[2 * j]) * p.gscale, f1 = __uint_as_float(v[2 * j + 1]) * p.gscale;
                        if (p.out_bf16) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(f0, f1);
                            o[j] = *reinterpret_cast<uint32_t*>(&h);
                        } else {
                            __half2 h = sat_half2(f0, f1);
                            o[j] = *reinterpret_cast<uint32_t*>(&h);
                        }
                    }
                };
                {
                    uint32_t v0[32], v1[32];
                    tmem_ld_32x32(tq, v0);
#pragma unroll
                    for (int ch = 0; ch < NV_BN / 32; ch += 2) {
                        tmem_ld_wait();
                        tmem_ld_32x32(tq + (uint32_t)(32 * (ch + 1)), v1);
                        pack(v0, w[ch]);
                        tmem_ld_wait();
                        if (ch + 2 < NV_BN / 32) tmem_ld_32x32(tq + (uint32_t)(32 * (ch + 2)), v0);
                        pack(v1, w[ch + 1]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_a(acce);                                        // this warp has read its quarter of the accumulator
#pragma unroll
                for (int ch = 0; ch < NV_BN / 32; ++ch) {
                    const int c = 32 * ch;
                    if (p.wide)
                        epilogue_stage_store_wide(outs, p.nout, stg, lane, w[ch], ch & 1, p.col0 + n0 + (c & ~63), row0, !failed && row0 < p.m && n0 + (c & ~63) < p.n);
                    else
                        epilogue_stage_store(outs, p.nout, stg, lane, w[ch], p.col0 + n0 + c, row0, !failed && row0 < p.m && n0 + c < p.n);
                }
                continue;
            } else {
            const int row = m0 + q * 32 + lane;
            const size_t doff = (size_t)row * p.ldd + n0;
            const bool vec = (p.ldd & 7) == 0;
#pragma unroll 1
            for (int c = 0; c < NV_BN; c += 32) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c, v);
                tmem_ld_wait();
                if (row < p.m && !failed) {
                    if (vec && n0 + c + 32 <= p.n) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint32_t w[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float f0 = __uint_as_float(v[j + 2 * e]) * p.gscale, f1 = __uint_as_float(v[j + 2 * e + 1]) * p.gscale;
                                if (p.out_bf16) {
                                    __nv_bfloat162 h = __floats2bfloat162_rn(f0, f1);
                                    w[e] = *reinterpret_cast<uint32_t*>(&h);
                                } else {
                                    __half2 h = sat_half2(f0, f1);
                                    w[e] = *reinterpret_cast<uint32_t*>(&h);
                                }
                            }
                            for (int pr = 0; pr < p.nout; ++pr) *reinterpret_cast<uint4*>(p.d[pr] + doff + c + j) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (n0 + c + j >= p.n) break;
                            const float f = __uint_as_float(v[j]) * p.gscale;
                            for (int pr = 0; pr < p.nout; ++pr) {
                                if (p.out_bf16) reinterpret_cast<__nv_bfloat16*>(p.d[pr])[doff + c + j] = __float2bfloat16_rn(f);
                                else p.d[pr][doff + c + j] = sat_half(f);
                            }
                        }
                    }
                }
            }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_a(acce);
        }
    }
    if (warp >= 2 && lane == 0 && p.tma_out) tma_store_wait_all();                 // the staging buffer must outlive its stores
    if (failed) atomicExch(p.status, KYB_DEV_TIMEOUT_GEMM);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}


// ------------------------------------------------------------------------------------------------ the same product by CTA pairs (tcgen05 cta_group::2)
// A cluster of two CTAs on neighbouring SMs computes a 256 x 256 tile: each CTA holds 128 rows of A and ONE HALF (128 rows) of the B tile in its shared memory,
// and a single MMA instruction issued by the pair's leader (cluster rank 0) runs on both tensor cores, each reading its own A rows and both halves of B. Per SM
// the B operand bytes written by TMA and read by the MMA are halved, which is what bounds the one-CTA kernel above (shared-memory bandwidth). Protocol:
//   full[s]   lives in the leader: one arrival (the leader's producer, with the byte count of BOTH CTAs' loads); every load of either CTA completes on it
//             (cp.async.bulk.tensor ... cta_group::2 with the leader's barrier address; no multicast anywhere)
//   empty[s]  lives in each CTA: the leader's tcgen05.commit arrives on both (commit multicast to the pair)
//   accf      in each CTA (commit multicast): the accumulator of the tile is complete; acce in the leader: 8 arrivals, the 4 epilogue warps of each CTA
// Scale factors: every CTA loads the chunks of its own 128 A rows and of ALL 256 B rows (4 KB per stage; both tensor cores need every column's scales), as tiled
// loads through two more tensor maps over the SF512 arrays, and tcgen05.cp cta_group::2 moves them into the tensor memory of both CTAs.
// Every wait is bounded; the pair meets at a cluster barrier before tensor memory is freed, so neither CTA leaves while the other can still signal it.
constexpr int NP_STAGES = 5;
constexpr uint32_t NP_A_BYTES = 128 * NV_BK / 2, NP_B_BYTES = 128 * NV_BK / 2, NP_STAGE_BYTES = NP_A_BYTES + NP_B_BYTES + NV_SFA_BYTES + NV_SFB_BYTES;   // 16 K + 16 K + 2 K + 4 K

__device__ __forceinline__ void tmem_cp_32x128b_x4_pair(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma_nvf4_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t tsfa, uint32_t tsfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(tsfa), "r"(tsfb), "r"(accumulate)
        : "memory");
}
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NV_THREADS, 1)
    gemm_nvfp4_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const __grid_constant__ CUtensorMap tma_sfa,
                           const __grid_constant__ CUtensorMap tma_sfb, const __grid_constant__ KybOutMaps outs, const NvGemmParams p, const int tiles_n, const int num_tiles) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    constexpr int STAGES = NP_STAGES;
    const uint32_t stg0 = smem0 + STAGES * NP_STAGE_BYTES;                         // epilogue staging, 4 warps
    const uint32_t bars = stg0 + 4 * KYB_STG_BYTES;
    const uint32_t full0 = bars, empty0 = bars + 8 * STAGES, accf = bars + 16 * STAGES, acce = accf + 8, tmem_slot = acce + 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair = (int)(blockIdx.x >> 1), pairs = (int)(gridDim.x >> 1);
    const int kblocks = p.k / NV_BK, k64 = p.k / 64;
    const int tiles_m = num_tiles / tiles_n;                                       // 256-row tiles
    constexpr uint32_t TMEM_COLS = 512, COL_SFA = 256, COL_SFB = 272;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init_a(full0 + 8 * s, 1), mbar_init_a(empty0 + 8 * s, 1);
        mbar_init_a(accf, 1);
        mbar_init_a(acce, 8);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&tma_a);
        prefetch_tmap(&tma_b);
        prefetch_tmap(&tma_sfa);
        prefetch_tmap(&tma_sfb);
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tc_fence_before();
    cluster_sync_all();                                                            // both CTAs' barriers exist before either signals the other
    tc_fence_after();
    const uint32_t tmem_base = lds32(tmem_slot);
    bool failed = false;

    if (warp == 0) {
        if (elect_one()) {
            uint32_t parity = 1;
            int s = 0;
            for (int t = pair; t < num_tiles && !failed; t += pairs) {
                const int n0 = (t / tiles_m) * NV_BN, m0 = (t % tiles_m) * 256 + (int)rank * 128;      // m fastest; this CTA's 128 rows of the tile
                for (int kb = 0; kb < kblocks && !failed; ++kb) {
                    if (!mbar_wait_fast(empty0 + 8 * s, parity)) failed = true;
                    const uint32_t a_dst = smem0 + s * NP_STAGE_BYTES, b_dst = a_dst + NP_A_BYTES, sfa_dst = b_dst + NP_B_BYTES, sfb_dst = sfa_dst + NV_SFA_BYTES;
                    if (rank == 0) mbar_expect_tx_a(full0 + 8 * s, 2 * NP_STAGE_BYTES);
                    const uint32_t bar = map_to_rank(full0 + 8 * s, 0);
                    tma_load_2d_pair(a_dst, &tma_a, kb * (NV_BK / 2), m0, bar);
                    tma_load_2d_pair(b_dst, &tma_b, kb * (NV_BK / 2), n0 + (int)rank * 128, bar);   // this CTA's half of the B tile
                    tma_load_2d_pair(sfa_dst, &tma_sfa, 0, (m0 >> 7) * k64 + kb * 4, bar);
                    tma_load_2d_pair(sfb_dst, &tma_sfb, 0, (n0 >> 7) * k64 + kb * 4, bar);
                    tma_load_2d_pair(sfb_dst + 2048, &tma_sfb, 0, ((n0 >> 7) + 1) * k64 + kb * 4, bar);
                    if (++s == STAGES) s = 0, parity ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        if (rank == 0 && elect_one()) {
            constexpr uint32_t idesc = umma_idesc_nvf4(256, NV_BN);
            uint32_t parity = 0;
            int s = 0, it = 0;
            for (int t = pair; t < num_tiles && !failed; t += pairs, ++it) {
                if (!mbar_wait_fast(acce, ((uint32_t)it & 1u) ^ 1u)) failed = true;         // both CTAs' epilogues have read the accumulator
                tc_fence_after();
                for (int kb = 0; kb < kblocks && !failed; ++kb) {
                    if (!mbar_wait_fast(full0 + 8 * s, parity)) failed = true;
                    tc_fence_after();
                    const uint32_t a_src = smem0 + s * NP_STAGE_BYTES, b_src = a_src + NP_A_BYTES, sfa_src = b_src + NP_B_BYTES, sfb_src = sfa_src + NV_SFA_BYTES;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        tmem_cp_32x128b_x4_pair(tmem_base + COL_SFA + 4 * j, sf_desc(sfa_src + 512 * j));
                        tmem_cp_32x128b_x4_pair(tmem_base + COL_SFB + 8 * j, sf_desc(sfb_src + 512 * j));
                        tmem_cp_32x128b_x4_pair(tmem_base + COL_SFB + 8 * j + 4, sf_desc(sfb_src + 2048 + 512 * j));
                    }
                    const uint64_t adesc = umma_desc_sw128(a_src), bdesc = umma_desc_sw128(b_src);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        umma_nvf4_pair(tmem_base, adesc + 2 * j, bdesc + 2 * j, idesc, tmem_base + COL_SFA + 4 * j, tmem_base + COL_SFB + 8 * j, (kb | j) != 0);
                    umma_commit_pair(empty0 + 8 * s);
                    if (++s == STAGES) s = 0, parity ^= 1u;
                }
                umma_commit_pair(accf);
            }
        }
    } else {
        const int q = warp & 3;
        const uint32_t acce_leader = map_to_rank(acce, 0);
        int it = 0;
        for (int t = pair; t < num_tiles; t += pairs, ++it) {
            const int n0 = (t / tiles_m) * NV_BN, m0 = (t % tiles_m) * 256 + (int)rank * 128;
            if (!mbar_wait_fast(accf, (uint32_t)it & 1u)) failed = true;
            tc_fence_after();
            const uint32_t stg = stg0 + (uint32_t)q * KYB_STG_BYTES;
            const int row0 = m0 + q * 32;
            const uint32_t tq = tmem_base + ((uint32_t)(q * 32) << 16);
            uint32_t w[NV_BN / 32][16];
            auto pack = [&](const uint32_t (&v)[32], uint32_t (&o)[16]) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float f0 = __uint_as_float(v[2 * j]) * p.gscale, f1 = __uint_as_float(v[2 * j + 1]) * p.gscale;
                    if (p.out_bf16) {
                        __nv_bfloat162 h = __floats2bfloat162_rn(f0, f1);
                        o[j] = *reinterpret_cast<uint32_t*>(&h);
                    } else {
                        __half2 h = sat_half2(f0, f1);
                        o[j] = *reinterpret_cast<uint32_t*>(&h);
                    }
                }
            };
            {
                uint32_t v0[32], v1[32];
                tmem_ld_32x32(tq, v0);
#pragma unroll
                for (int ch = 0; ch < NV_BN / 32; ch += 2) {
                    tmem_ld_wait();
                    tmem_ld_32x32(tq + (uint32_t)(32 * (ch + 1)), v1);
                    pack(v0, w[ch]);
                    tmem_ld_wait();
                    if (ch + 2 < NV_BN / 32) tmem_ld_32x32(tq + (uint32_t)(32 * (ch + 2)), v0);
                    pack(v1, w[ch + 1]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acce_leader);                               // this warp has read its quarter of this CTA's accumulator
#pragma unroll
            for (int ch = 0; ch < NV_BN / 32; ++ch)
                epilogue_stage_store(outs, 1, stg, lane, w[ch], n0 + 32 * ch, row0, !failed && row0 < p.m);
        }
    }
    if (warp >= 2 && lane == 0) tma_store_wait_all();                              // the staging buffer must outlive its stores
    if (failed) atomicExch(p.status, KYB_DEV_TIMEOUT_GEMM);
    tc_fence_before();
    cluster_sync_all();                                                            // neither CTA frees tensor memory or leaves while the other may still signal it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

}  // namespace kyb

// ------------------------------------------------------------------------------------------------ host side
extern "C" size_t kyb_nvfp4_sf_bytes(int64_t rows, int64_t k) {
    if (rows <= 0 || k <= 0 || k % 64) return 0;
    return (size_t)((rows + 127) / 128) * (size_t)(k / 64) * 512;
}

extern "C" int kyb_nvfp4_quant_rows(const void* x, int x_dtype, int64_t ldx, int64_t rows, int64_t k, void* codes, void* sf_plain, void* sf_swz, void* stream) {
    KYB_REQUIRE(x && codes && (sf_plain || sf_swz), "null pointer");
    KYB_REQUIRE(rows > 0 && k > 0 && k % 16 == 0 && ldx >= k, "rows=%lld k=%lld: k must be a positive multiple of 16", (long long)rows, (long long)k);
    KYB_REQUIRE(!sf_swz || k % 64 == 0, "the tensor-core scale layout needs k %% 64 == 0");
    KYB_REQUIRE(x_dtype == 1 || x_dtype == 2, "x_dtype: 1 = fp16, 2 = bf16");
    KYB_REQUIRE(((uintptr_t)codes & 7) == 0, "codes must be 8-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    if (sf_swz && rows % 128) KYB_CUDA(cudaMemsetAsync(sf_swz, 0, kyb_nvfp4_sf_bytes(rows, k), st));   // padding rows of the last 128-row block read as zero scales
    if (k % 64 == 0 && ldx % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)codes & 15) == 0 && (!sf_plain || ((uintptr_t)sf_plain & 3) == 0)) {
        const int64_t blocks16 = rows * (k / 16);
        const unsigned gb = (unsigned)((blocks16 + 255) / 256);
        if (x_dtype == 1) kyb::nvfp4_quant_rows_kernel<__half><<<gb, 256, 0, st>>>((const __half*)x, ldx, rows, k, (uint8_t*)codes, (uint8_t*)sf_plain, (uint8_t*)sf_swz);
        else kyb::nvfp4_quant_rows_kernel<__nv_bfloat16><<<gb, 256, 0, st>>>((const __nv_bfloat16*)x, ldx, rows, k, (uint8_t*)codes, (uint8_t*)sf_plain, (uint8_t*)sf_swz);
        return kyb_launch_check("nvfp4_quant_rows");
    }
    const int64_t total = rows * (k / 16);
    const unsigned blocks = (unsigned)((total + 127) / 128);
    if (x_dtype == 1) kyb::nvfp4_quant_rows16_kernel<__half><<<blocks, 128, 0, st>>>((const __half*)x, ldx, rows, k, (uint8_t*)codes, (uint8_t*)sf_plain, (uint8_t*)sf_swz);
    else kyb::nvfp4_quant_rows16_kernel<__nv_bfloat16><<<blocks, 128, 0, st>>>((const __nv_bfloat16*)x, ldx, rows, k, (uint8_t*)codes, (uint8_t*)sf_plain, (uint8_t*)sf_swz);
    return kyb_launch_check("nvfp4_quant_rows");
}

extern "C" int kyb_nvfp4_unpack_rows(const void* codes, const void* sf_plain, int64_t rows, int64_t k, int out_dtype, void* out, int64_t ldo, void* stream) {
    KYB_REQUIRE(codes && sf_plain && out, "null pointer");
    KYB_REQUIRE(rows > 0 && k > 0 && k % 16 == 0 && ldo >= k, "rows=%lld k=%lld", (long long)rows, (long long)k);
    KYB_REQUIRE(out_dtype >= 0 && out_dtype <= 2, "out_dtype: 0 = fp32, 1 = fp16, 2 = bf16");
    const int64_t total = rows * (k / 16);
    const unsigned blocks = (unsigned)((total + 127) / 128);
    cudaStream_t st = (cudaStream_t)stream;
    if (out_dtype == 0) kyb::nvfp4_unpack_rows_kernel<float><<<blocks, 128, 0, st>>>((const uint8_t*)codes, (const uint8_t*)sf_plain, rows, k, (float*)out, ldo);
    else if (out_dtype == 1) kyb::nvfp4_unpack_rows_kernel<__half><<<blocks, 128, 0, st>>>((const uint8_t*)codes, (const uint8_t*)sf_plain, rows, k, (__half*)out, ldo);
    else kyb::nvfp4_unpack_rows_kernel<__nv_bfloat16><<<blocks, 128, 0, st>>>((const uint8_t*)codes, (const uint8_t*)sf_plain, rows, k, (__nv_bfloat16*)out, ldo);
    return kyb_launch_check("nvfp4_unpack_rows");
}

extern "C" int kyb_fp4_quant_block32(const void* x, int x_dtype, int64_t ldx, int64_t rows, int64_t k, void* codes, void* sbytes, void* stream) {
    KYB_REQUIRE(x && codes && sbytes, "null pointer");
    KYB_REQUIRE(x_dtype == KYB_DT_F16 || x_dtype == KYB_DT_BF16, "x dtype %d: fp16 or bf16", x_dtype);
    KYB_REQUIRE(rows > 0 && k > 0 && k % 32 == 0 && ldx >= k, "rows=%lld k=%lld: k must be a positive multiple of 32", (long long)rows, (long long)k);
    const int64_t total = rows * (k / 32);
    const unsigned blocks = (unsigned)((total + 127) / 128);
    cudaStream_t st = (cudaStream_t)stream;
    if (x_dtype == KYB_DT_F16) kyb::fp4_quant_block32_kernel<__half><<<blocks, 128, 0, st>>>((const __half*)x, ldx, rows, k, (uint8_t*)codes, (uint8_t*)sbytes);
    else kyb::fp4_quant_block32_kernel<__nv_bfloat16><<<blocks, 128, 0, st>>>((const __nv_bfloat16*)x, ldx, rows, k, (uint8_t*)codes, (uint8_t*)sbytes);
    return kyb_launch_check("fp4_quant_block32");
}

extern "C" int kyb_fp4_unpack_block32(const void* codes, const void* sbytes, int64_t rows, int64_t k, int out_dtype, void* out, int64_t ldo, void* stream) {
    KYB_REQUIRE(codes && sbytes && out, "null pointer");
    KYB_REQUIRE(rows > 0 && k > 0 && k % 32 == 0 && ldo >= k && out_dtype >= 0 && out_dtype <= 2, "rows=%lld k=%lld out_dtype=%d", (long long)rows, (long long)k, out_dtype);
    KYB_REQUIRE(((uintptr_t)codes & 15) == 0, "codes must be 16-byte aligned");
    const int64_t total = rows * (k / 32);
    const unsigned blocks = (unsigned)((total + 127) / 128);
    cudaStream_t st = (cudaStream_t)stream;
    if (out_dtype == 0) kyb::fp4_unpack_block32_kernel<float><<<blocks, 128, 0, st>>>((const uint8_t*)codes, (const uint8_t*)sbytes, rows, k, (float*)out, ldo);
    else if (out_dtype == 1) kyb::fp4_unpack_block32_kernel<__half><<<blocks, 128, 0, st>>>((const uint8_t*)codes, (const uint8_t*)sbytes, rows, k, (__half*)out, ldo);
    else kyb::fp4_unpack_block32_kernel<__nv_bfloat16><<<blocks, 128, 0, st>>>((const uint8_t*)codes, (const uint8_t*)sbytes, rows, k, (__nv_bfloat16*)out, ldo);
    return kyb_launch_check("fp4_unpack_block32");
}

extern "C" int kyb_nvfp4_sf_swizzle(void* plain, int64_t rows, int64_t k, void* swz, int to_swizzled, void* stream) {
    KYB_REQUIRE(plain && swz, "null pointer");
    KYB_REQUIRE(rows > 0 && k > 0 && k % 64 == 0, "rows=%lld k=%lld: k must be a positive multiple of 64", (long long)rows, (long long)k);
    const int64_t total = ((rows + 127) / 128 * 128) * (k / 16);
    kyb::sf_swizzle_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint8_t*)plain, rows, k, (uint8_t*)swz, to_swizzled);
    return kyb_launch_check("nvfp4_sf_swizzle");
}

// D [m, n] = sat(gscale * A B^T): a_codes [m, k/2], b_codes [n, k/2] packed e2m1 (two per byte, low nibble first), sfa / sfb in the SF512 layout.
static int nvfp4_gemm_impl(const void* a_codes, const void* sfa, const void* b_codes, const void* sfb, int64_t m, int64_t n, int64_t k, float gscale, int out_dtype,
                           void* const* d, int nout, int64_t ldd, int64_t col0, void* stream, bool pair_ok = true) {
    KYB_REQUIRE(a_codes && sfa && b_codes && sfb, "null pointer");
    KYB_REQUIRE(m > 0 && n > 0 && k > 0 && k % 256 == 0, "m=%lld n=%lld k=%lld: k must be a positive multiple of 256", (long long)m, (long long)n, (long long)k);
    KYB_REQUIRE(n % 256 == 0, "n=%lld must be a multiple of 256 (one CTA covers two 128-row scale chunks of B)", (long long)n);
    KYB_REQUIRE(ldd >= n && (out_dtype == 1 || out_dtype == 2), "ldd >= n, out_dtype 1 = fp16 or 2 = bf16");
    KYB_REQUIRE(((uintptr_t)a_codes & 15) == 0 && ((uintptr_t)b_codes & 15) == 0 && ((uintptr_t)sfa & 15) == 0 && ((uintptr_t)sfb & 15) == 0, "operands must be 16-byte aligned");
    unsigned int* status = kyb_device_status_word();
    KYB_REQUIRE(status, "could not set up the device status word");
    CUtensorMap ta, tb;
    if (int rc = kyb_make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_codes, (uint64_t)m, (uint64_t)(k / 2), (uint64_t)(k / 2), kyb::NV_BM, 128)) return rc;
    if (int rc = kyb_make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b_codes, (uint64_t)n, (uint64_t)(k / 2), (uint64_t)(k / 2), kyb::NV_BN, 128)) return rc;
    kyb::NvGemmParams p;
    p.sfa = (const uint8_t*)sfa, p.sfb = (const uint8_t*)sfb, p.ldd = ldd, p.m = (int)m, p.n = (int)n, p.k = (int)k, p.gscale = gscale;
    p.out_bf16 = out_dtype == 2, p.status = status, p.nout = nout;
    for (int i = 0; i < 8; ++i) p.d[i] = i < nout ? (__half*)d[i] + col0 : nullptr;
    KybOutMaps outs;
    memset(&outs, 0, sizeof(outs));
    p.col0 = (int)col0;
    p.tma_out = (ldd % 8 == 0 && col0 % 8 == 0) ? 1 : 0;                            // tiled bulk stores need 16-byte aligned bases and row pitches
    for (int i = 0; i < nout && p.tma_out; ++i)
        if ((uintptr_t)d[i] & 15) p.tma_out = 0;
    p.wide = (p.tma_out && nout > 1) ? 1 : 0;
    p.stages = p.wide ? kyb::NV_STAGES - 1 : kyb::NV_STAGES;
    for (int i = 0; i < nout && p.tma_out; ++i)
        if (int rc = kyb_make_tmap_2d(&outs.m[i], CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, d[i], (uint64_t)m, (uint64_t)(col0 + n), (uint64_t)ldd * 2, 32, p.wide ? 64 : 32,
                                      p.wide ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B))
            return rc;
    int dev = 0;
    KYB_CUDA(cudaGetDevice(&dev));
    static std::mutex mu;
    if (nout == 1 && p.tma_out && m > 128 && pair_ok) {
        // one destination and at least two row blocks: CTA pairs (cta_group::2), each CTA holding half of the B tile
        CUtensorMap tbh, tsa, tsb;
        const uint64_t k64 = (uint64_t)(k / 64);
        if (int rc = kyb_make_tmap_2d(&tbh, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b_codes, (uint64_t)n, (uint64_t)(k / 2), (uint64_t)(k / 2), 128, 128)) return rc;
        if (int rc = kyb_make_tmap_2d(&tsa, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, sfa, (uint64_t)((m + 127) / 128) * k64, 128, 512, 4, 128, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
        if (int rc = kyb_make_tmap_2d(&tsb, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, sfb, (uint64_t)(n / 128) * k64, 128, 512, 4, 128, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
        constexpr size_t psmem = (size_t)kyb::NP_STAGES * kyb::NP_STAGE_BYTES + 4 * KYB_STG_BYTES + 16 * kyb::NP_STAGES + 32 + 1024;
        static unsigned pdone = 0;
        static int pairs_max[32] = {0};
        {
            std::lock_guard<std::mutex> lk(mu);
            if (!(pdone & (1u << (dev & 31)))) {
                KYB_CUDA(cudaFuncSetAttribute(kyb::gemm_nvfp4_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)psmem));
                // how many pairs the device can hold at once (one CTA per SM, pairs on neighbouring SMs)
                cudaLaunchConfig_t qc = {};
                qc.gridDim = dim3(2), qc.blockDim = dim3(kyb::NV_THREADS), qc.dynamicSmemBytes = psmem;
                int nc = 0;
                if (cudaOccupancyMaxActiveClusters(&nc, kyb::gemm_nvfp4_pair_kernel, &qc) != cudaSuccess || nc <= 0) {
                    (void)cudaGetLastError();
                    nc = 0;
                }
                pairs_max[dev & 31] = nc;
                pdone |= 1u << (dev & 31);
            }
        }
        const int pm = pairs_max[dev & 31];
        const int pair_tiles = (int)(n / kyb::NV_BN) * (int)((m + 255) / 256);
        // more tiles than pairs but no more than SMs: the one-CTA kernel (twice as many, half as large tiles) fills the device better than a second, short wave of pairs
        if (pm > 0 && !(pair_tiles > pm && pair_tiles <= 2 * pm)) {
            const int tiles_n = (int)(n / kyb::NV_BN), num_tiles = tiles_n * (int)((m + 255) / 256);
            const int pairs = num_tiles < pm ? num_tiles : pm;
            kyb::gemm_nvfp4_pair_kernel<<<(unsigned)(2 * pairs), kyb::NV_THREADS, psmem, (cudaStream_t)stream>>>(ta, tbh, tsa, tsb, outs, p, tiles_n, num_tiles);
            return kyb_launch_check("gemm_nvfp4_pair");
        }
    }
    const size_t smem = (size_t)p.stages * kyb::NV_STAGE_BYTES + 4 * (p.wide ? 2 : 1) * KYB_STG_BYTES + 16 * kyb::NV_STAGES + 32 + 1024;
    constexpr size_t smem_max = (size_t)kyb::NV_STAGES * kyb::NV_STAGE_BYTES + 4 * KYB_STG_BYTES + 16 * kyb::NV_STAGES + 32 + 1024;
    static unsigned done = 0;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!(done & (1u << (dev & 31)))) {
            KYB_CUDA(cudaFuncSetAttribute(kyb::gemm_nvfp4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
            done |= 1u << (dev & 31);
        }
    }
    int sms = 148;
    KYB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int tiles_n = (int)((n + kyb::NV_BN - 1) / kyb::NV_BN), num_tiles = tiles_n * (int)((m + kyb::NV_BM - 1) / kyb::NV_BM);
    kyb::gemm_nvfp4_kernel<<<(unsigned)(num_tiles < sms ? num_tiles : sms), kyb::NV_THREADS, smem, (cudaStream_t)stream>>>(ta, tb, outs, p, tiles_n, num_tiles);
    return kyb_launch_check("gemm_nvfp4");
}

extern "C" int kyb_gemm_nvfp4(const void* a_codes, const void* sfa, const void* b_codes, const void* sfb, int64_t m, int64_t n, int64_t k, float gscale, int out_dtype,
                              void* d, int64_t ldd, void* stream) {
    KYB_REQUIRE(d, "null pointer");
    void* outs[1] = {d};
    return nvfp4_gemm_impl(a_codes, sfa, b_codes, sfb, m, n, k, gscale, out_dtype, outs, 1, ldd, 0, stream);
}

// The same product with the all-gather of an N-sharded linear folded into the epilogue: every tile goes to the output matrix of every rank, at column col0.
extern "C" int kyb_gemm_nvfp4_ag(const void* a_codes, const void* sfa, const void* b_codes, const void* sfb, int64_t m, int64_t n, int64_t k, float gscale, int out_dtype,
                                 const kyb_peer_out* out, int64_t ldd, int64_t col0, void* stream) {
    KYB_REQUIRE(out && out->count >= 1 && out->count <= 8, "peer outputs: 1..8 ranks");
    KYB_REQUIRE(col0 >= 0 && col0 % 8 == 0 && col0 + n <= ldd && ldd % 8 == 0, "col0=%lld: a multiple of 8 with col0 + n <= ldd, ldd a multiple of 8", (long long)col0);
    void* outs[8];
    for (int i = 0; i < out->count; ++i) {
        KYB_REQUIRE(out->ptr[i] && ((uintptr_t)out->ptr[i] & 15) == 0, "peer output %d is null or not 16-byte aligned", i);
        outs[i] = out->ptr[i];
    }
    return nvfp4_gemm_impl(a_codes, sfa, b_codes, sfb, m, n, k, gscale, out_dtype, outs, out->count, ldd, col0, stream);
}
