// Decode GEMV / few-row product on T16 weights: y[m, n] = x[m, k] W[n, k]^T for m <= 32.
//
// HBM-bound design. One warp owns one 16-row tile over a k-part and streams its tiles (contiguous in T16) through a private
// ring of bulk copies (cp.async.bulk -> shared memory, mbarrier completion), so the bytes in flight do not depend on
// registers. Lane (g, t) reads its 16-byte units with LDS.128, unpacks the 4/6/3-bit fields with a few LOP3/PRMT into fp16
// operand registers and feeds mma.sync.m16n8k16 (weights = A, activations = B, fp32 accumulate): the integer codes are
// exact in fp16 and every product code * x is exact in fp32; the block scales are applied in fp32 to the 16- or 32-input
// partial sums, so no weight is ever rounded. The tensor-core instruction is used because at ~7 TB/s a scalar fp32
// FMA per weight and activation row exceeds the SM's issue rate (about 3 issue slots per 4-bit weight are available);
// with mma the cost per weight is independent of m up to 8 rows per column tile.
// The activations of the k-part are staged once per CTA as ready-made B fragments. Split-k partials (fp32) go to a
// caller-provided workspace and are summed in a fixed order by the finalize kernel, so results are deterministic and the
// result of an activation row does not depend on how many rows ride along.
#include <algorithm>
#include <atomic>

#include "t16_decode.cuh"

#ifndef KYB_Q4K_SUBNORMAL
#define KYB_Q4K_SUBNORMAL 1   // 1: 4-bit codes enter the MMA as fp16 subnormals (code * 2^-24), 0: as 1024 + code minus 1024
#endif

namespace kyb {

struct GemvParams {
    const uint8_t* t16;
    const __half* x;
    __half* y;
    float* partial;          // [ksplit][mpad][npad] when ksplit > 1
    unsigned int* status;
    int64_t ldx, ldy;
    int n, npad, nb;         // rows, rows padded to 16, k-blocks of 256
    int m, mst;              // activation rows, rows stored per column tile (1, 2, 4, 8)
    int kbp, ksplit;         // k-blocks per part, parts
    int warps, stages;
    float gscale;
};

constexpr int SCL_BYTES = 16 * 16 * 4;   // per-warp scale scratch: 16 rows x 16 floats

template <int FMT>
__host__ __device__ constexpr int xaux_bytes_per_block(int nt) { return FMT == KYB_FMT_Q4_K ? 256 * nt : 0; }

__device__ __forceinline__ uint32_t magic_sub(uint32_t h2_with_magic, uint32_t sub_bits) {
    __half2 a = *reinterpret_cast<__half2*>(&h2_with_magic), b = *reinterpret_cast<__half2*>(&sub_bits);
    __half2 r = __hsub2(a, b);
    return *reinterpret_cast<uint32_t*>(&r);
}

// ---- per-format: scale preparation (all lanes cooperate, results in scl[16][16] floats) ----------------------------------
template <int FMT>
__device__ __forceinline__ void prep_scales(const uint8_t* tile, float* scl, int lane) {
    const int r = lane >> 1, hf = lane & 1;
    if constexpr (FMT == KYB_FMT_Q4_K) {
        const uint4 mt = *reinterpret_cast<const uint4*>(tile + 2048 + r * 16);
        const uint32_t scw = hf ? ((mt.w & 0x0f0f0f0fu) | ((mt.y >> 2) & 0x30303030u)) : (mt.y & 0x3f3f3f3fu);
        const float d = half_bits_to_float(mt.x & 0xffffu);
#if KYB_Q4K_SUBNORMAL
        const float dlo = d * 16777216.0f, dhi = d * 1048576.0f;     // even sub-blocks: code * 2^-24, odd: code * 2^-20
#else
        const float dlo = d, dhi = d * 0.0625f;
#endif
        float4 o;
        o.x = dlo * (float)(scw & 255u);
        o.y = dhi * (float)((scw >> 8) & 255u);
        o.z = dlo * (float)((scw >> 16) & 255u);
        o.w = dhi * (float)(scw >> 24);
        *reinterpret_cast<float4*>(scl + r * 16 + 4 * hf) = o;
    } else if constexpr (FMT == KYB_FMT_Q6_K) {
        const uint2 sw = *reinterpret_cast<const uint2*>(tile + 3072 + r * 16 + 8 * hf);
        const float d = ldh(tile + 3328 + r * 2);
        float4 a, b;
        a.x = d * (float)(int)(int8_t)(sw.x & 255u);
        a.y = d * (float)(int)(int8_t)((sw.x >> 8) & 255u);
        a.z = d * (float)(int)(int8_t)((sw.x >> 16) & 255u);
        a.w = d * (float)(int)(int8_t)(sw.x >> 24);
        b.x = d * (float)(int)(int8_t)(sw.y & 255u);
        b.y = d * (float)(int)(int8_t)((sw.y >> 8) & 255u);
        b.z = d * (float)(int)(int8_t)((sw.y >> 16) & 255u);
        b.w = d * (float)(int)(int8_t)(sw.y >> 24);
        *reinterpret_cast<float4*>(scl + r * 16 + 8 * hf) = a;
        *reinterpret_cast<float4*>(scl + r * 16 + 8 * hf + 4) = b;
    } else if constexpr (FMT == KYB_FMT_Q3_K) {
        const uint8_t* sp = tile + 1536 + r * 12;
        const uint32_t w0 = ldw(sp), w1 = ldw(sp + 4), w2 = ldw(sp + 8);
        const uint32_t ga = hf ? (((w0 >> 4) & 0x0f0f0f0fu) | (w2 & 0x30303030u)) : ((w0 & 0x0f0f0f0fu) | ((w2 << 4) & 0x30303030u));
        const uint32_t gb = hf ? (((w1 >> 4) & 0x0f0f0f0fu) | ((w2 >> 2) & 0x30303030u)) : ((w1 & 0x0f0f0f0fu) | ((w2 << 2) & 0x30303030u));
        const float d = ldh(tile + 1728 + r * 2);
        float4 a, b;
        a.x = d * (float)((int)(ga & 255u) - 32);
        a.y = d * (float)((int)((ga >> 8) & 255u) - 32);
        a.z = d * (float)((int)((ga >> 16) & 255u) - 32);
        a.w = d * (float)((int)(ga >> 24) - 32);
        b.x = d * (float)((int)(gb & 255u) - 32);
        b.y = d * (float)((int)((gb >> 8) & 255u) - 32);
        b.z = d * (float)((int)((gb >> 16) & 255u) - 32);
        b.w = d * (float)((int)(gb >> 24) - 32);
        *reinterpret_cast<float4*>(scl + r * 16 + 8 * hf) = a;
        *reinterpret_cast<float4*>(scl + r * 16 + 8 * hf + 4) = b;
    } else {
        const uint2 sw = *reinterpret_cast<const uint2*>(tile + 2048 + r * 16 + 8 * hf);
        float4 a, b;                                                   // e2m1 operands carry 2^-14: fold 2^14 here
        a.x = e4m3_unsigned(sw.x) * 16384.0f;
        a.y = e4m3_unsigned(sw.x >> 8) * 16384.0f;
        a.z = e4m3_unsigned(sw.x >> 16) * 16384.0f;
        a.w = e4m3_unsigned(sw.x >> 24) * 16384.0f;
        b.x = e4m3_unsigned(sw.y) * 16384.0f;
        b.y = e4m3_unsigned(sw.y >> 8) * 16384.0f;
        b.z = e4m3_unsigned(sw.y >> 16) * 16384.0f;
        b.w = e4m3_unsigned(sw.y >> 24) * 16384.0f;
        *reinterpret_cast<float4*>(scl + r * 16 + 8 * hf) = a;
        *reinterpret_cast<float4*>(scl + r * 16 + 8 * hf + 4) = b;
    }
}

template <int NT>
struct Acc {
    float v[NT][4];
};

// B fragments of one 16-input chunk for column tile nt (zero for lanes whose activation row is not stored)
__device__ __forceinline__ uint2 load_b(const uint8_t* xfrag, int chunk, int nt, int NT_, int mst, int g, int t) {
    uint2 b = make_uint2(0u, 0u);
    if (g < mst) b = *reinterpret_cast<const uint2*>(xfrag + ((size_t)(chunk * NT_ + nt) * mst + g) * 32 + t * 8);
    return b;
}

template <int NT>
__device__ __forceinline__ void scale_acc(Acc<NT>& acc, const float (&c)[NT][4], float s_lo, float s_hi) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        acc.v[nt][0] = fmaf(s_lo, c[nt][0], acc.v[nt][0]);
        acc.v[nt][1] = fmaf(s_lo, c[nt][1], acc.v[nt][1]);
        acc.v[nt][2] = fmaf(s_hi, c[nt][2], acc.v[nt][2]);
        acc.v[nt][3] = fmaf(s_hi, c[nt][3], acc.v[nt][3]);
    }
}

// ---- one tile (16 rows x 256 inputs) ----------------------------------------------------------------------------------
template <int FMT, int NT>
__device__ __forceinline__ void consume_tile(const uint8_t* tile, const float* scl, const uint8_t* xfrag, const uint8_t* xaux, int blk, int mst, int lane,
                                             Acc<NT>& acc) {
    const int g = lane >> 2, t = lane & 3;
    const int chunk0 = blk * 16;
    if constexpr (FMT == KYB_FMT_Q4_K) {
        // scales of rows g and g + 8 for the 8 sub-blocks
        const float4 s0a = *reinterpret_cast<const float4*>(scl + g * 16), s0b = *reinterpret_cast<const float4*>(scl + g * 16 + 4);
        const float4 s1a = *reinterpret_cast<const float4*>(scl + (g + 8) * 16), s1b = *reinterpret_cast<const float4*>(scl + (g + 8) * 16 + 4);
        const float sg[8] = {s0a.x, s0a.y, s0a.z, s0a.w, s0b.x, s0b.y, s0b.z, s0b.w};
        const float sh[8] = {s1a.x, s1a.y, s1a.z, s1a.w, s1b.x, s1b.y, s1b.z, s1b.w};
#pragma unroll
        for (int G = 0; G < 4; ++G) {
            const uint4 u = *reinterpret_cast<const uint4*>(tile + (G * 32 + lane) * 16);
            float clo[NT][4], chi[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) clo[nt][i] = 0.f, chi[nt][i] = 0.f;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const uint32_t wg = c ? u.z : u.x, wh = c ? u.w : u.y;
                const uint32_t wg8 = wg >> 8, wh8 = wh >> 8;
#if KYB_Q4K_SUBNORMAL
                const uint32_t l0 = wg & 0x000F000Fu, l1 = wh & 0x000F000Fu, l2 = wg8 & 0x000F000Fu, l3 = wh8 & 0x000F000Fu;
                const uint32_t h0 = wg & 0x00F000F0u, h1 = wh & 0x00F000F0u, h2 = wg8 & 0x00F000F0u, h3 = wh8 & 0x00F000F0u;
#else
                const uint32_t l0 = magic_sub(and_or(wg, 0x000F000Fu, 0x64006400u), 0x64006400u), l1 = magic_sub(and_or(wh, 0x000F000Fu, 0x64006400u), 0x64006400u);
                const uint32_t l2 = magic_sub(and_or(wg8, 0x000F000Fu, 0x64006400u), 0x64006400u), l3 = magic_sub(and_or(wh8, 0x000F000Fu, 0x64006400u), 0x64006400u);
                const uint32_t h0 = magic_sub(and_or(wg, 0x00F000F0u, 0x64006400u), 0x64006400u), h1 = magic_sub(and_or(wh, 0x00F000F0u, 0x64006400u), 0x64006400u);
                const uint32_t h2 = magic_sub(and_or(wg8, 0x00F000F0u, 0x64006400u), 0x64006400u), h3 = magic_sub(and_or(wh8, 0x00F000F0u, 0x64006400u), 0x64006400u);
#endif
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint2 bl = load_b(xfrag, chunk0 + 4 * G + c, nt, NT, mst, g, t);
                    mma16816(clo[nt], l0, l1, l2, l3, bl.x, bl.y);
                    const uint2 bh = load_b(xfrag, chunk0 + 4 * G + 2 + c, nt, NT, mst, g, t);
                    mma16816(chi[nt], h0, h1, h2, h3, bh.x, bh.y);
                }
            }
            scale_acc<NT>(acc, clo, sg[2 * G], sh[2 * G]);
            scale_acc<NT>(acc, chi, sg[2 * G + 1], sh[2 * G + 1]);
        }
        // minus dmin * sum_j mn_j * (sum of x over sub-block j): an m16n8k8 product of the 6-bit mins with the staged sums (fp16 hi + lo)
        const uint4 mg = *reinterpret_cast<const uint4*>(tile + 2048 + g * 16), mh = *reinterpret_cast<const uint4*>(tile + 2048 + (g + 8) * 16);
        const uint32_t mng = (t & 2) ? (((mg.w >> 4) & 0x0f0f0f0fu) | ((mg.z >> 2) & 0x30303030u)) : (mg.z & 0x3f3f3f3fu);
        const uint32_t mnh = (t & 2) ? (((mh.w >> 4) & 0x0f0f0f0fu) | ((mh.z >> 2) & 0x30303030u)) : (mh.z & 0x3f3f3f3fu);
        const uint32_t sel = (t & 1) ? 0x4342u : 0x4140u;
#if KYB_Q4K_SUBNORMAL
        const uint32_t a0 = prmt(mng, 0u, sel), a1 = prmt(mnh, 0u, sel);
        const float dmg = half_bits_to_float(mg.x >> 16) * 16777216.0f, dmh = half_bits_to_float(mh.x >> 16) * 16777216.0f;
#else
        const uint32_t a0 = magic_sub(prmt(mng, 0x64646464u, sel), 0x64006400u), a1 = magic_sub(prmt(mnh, 0x64646464u, sel), 0x64006400u);
        const float dmg = half_bits_to_float(mg.x >> 16), dmh = half_bits_to_float(mh.x >> 16);
#endif
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float tt[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t* xa = reinterpret_cast<const uint32_t*>(xaux + (size_t)blk * 256 * NT);
            mma1688(tt, a0, a1, xa[(0 * NT + nt) * 32 + lane]);
            mma1688(tt, a0, a1, xa[(1 * NT + nt) * 32 + lane]);
            acc.v[nt][0] = fmaf(-dmg, tt[0], acc.v[nt][0]);
            acc.v[nt][1] = fmaf(-dmg, tt[1], acc.v[nt][1]);
            acc.v[nt][2] = fmaf(-dmh, tt[2], acc.v[nt][2]);
            acc.v[nt][3] = fmaf(-dmh, tt[3], acc.v[nt][3]);
        }
    } else {
        // one scale per MMA slice s = 0..15
        float sg[16], sh[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 a = *reinterpret_cast<const float4*>(scl + g * 16 + 4 * q), b = *reinterpret_cast<const float4*>(scl + (g + 8) * 16 + 4 * q);
            sg[4 * q] = a.x, sg[4 * q + 1] = a.y, sg[4 * q + 2] = a.z, sg[4 * q + 3] = a.w;
            sh[4 * q] = b.x, sh[4 * q + 1] = b.y, sh[4 * q + 2] = b.z, sh[4 * q + 3] = b.w;
        }
        uint4 hi = make_uint4(0, 0, 0, 0), hb = make_uint4(0, 0, 0, 0);
        if constexpr (FMT == KYB_FMT_Q3_K) hb = *reinterpret_cast<const uint4*>(tile + 1024 + lane * 16);
#pragma unroll
        for (int P = 0; P < 4; ++P) {
            uint4 u;
            if constexpr (FMT == KYB_FMT_Q6_K) {
                u = *reinterpret_cast<const uint4*>(tile + (P * 32 + lane) * 16);
                if ((P & 1) == 0) hi = *reinterpret_cast<const uint4*>(tile + 2048 + ((P >> 1) * 32 + lane) * 16);
            } else if constexpr (FMT == KYB_FMT_Q3_K) {
                if ((P & 1) == 0) hi = *reinterpret_cast<const uint4*>(tile + ((P >> 1) * 32 + lane) * 16);     // 2-bit plane
                u = hi;
            } else {
                u = *reinterpret_cast<const uint4*>(tile + (P * 32 + lane) * 16);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {                                 // s = 4 P + i
                const int s = 4 * P + i;
                uint32_t a0, a1, a2, a3;
                if constexpr (FMT == KYB_FMT_Q6_K) {
                    const int p = i >> 1;
                    uint32_t wg = p ? u.z : u.x, wh = p ? u.w : u.y;
                    if (i & 1) wg >>= 4, wh >>= 4;
                    uint32_t hg = (P & 1) ? hi.z : hi.x, hh = (P & 1) ? hi.w : hi.y;
                    if (i == 0) hg <<= 4, hh <<= 4;
                    else if (i == 1) hg <<= 2, hh <<= 2;
                    else if (i == 3) hg >>= 2, hh >>= 2;
                    const uint32_t vg = and_or(wg, 0x0F0F0F0Fu, hg & 0x30303030u), vh = and_or(wh, 0x0F0F0F0Fu, hh & 0x30303030u);
                    // bytes -> fp16 (1024 + v) - 1056 = v - 32, exact
                    a0 = magic_sub(prmt(vg, 0x64646464u, 0x4240u), 0x64206420u);
                    a2 = magic_sub(prmt(vg, 0x64646464u, 0x4341u), 0x64206420u);
                    a1 = magic_sub(prmt(vh, 0x64646464u, 0x4240u), 0x64206420u);
                    a3 = magic_sub(prmt(vh, 0x64646464u, 0x4341u), 0x64206420u);
                } else if constexpr (FMT == KYB_FMT_Q3_K) {
                    uint32_t wg = (P & 1) ? u.z : u.x, wh = (P & 1) ? u.w : u.y;     // word a = (s >> 2) & 1 = P & 1
                    wg >>= 2 * i, wh >>= 2 * i;
                    uint32_t bg = (P & 2) ? hb.z : hb.x, bh = (P & 2) ? hb.w : hb.y;   // word a' = s >> 3
                    const int i8 = s & 7;                                               // bit i8 -> bit 2
                    if (i8 < 2) bg <<= (2 - i8), bh <<= (2 - i8);
                    else bg >>= (i8 - 2), bh >>= (i8 - 2);
                    const uint32_t vg = and_or(wg, 0x03030303u, bg & 0x04040404u), vh = and_or(wh, 0x03030303u, bh & 0x04040404u);
                    // (1024 + v) - 1028 = v - 4
                    a0 = magic_sub(prmt(vg, 0x64646464u, 0x4240u), 0x64046404u);
                    a2 = magic_sub(prmt(vg, 0x64646464u, 0x4341u), 0x64046404u);
                    a1 = magic_sub(prmt(vh, 0x64646464u, 0x4240u), 0x64046404u);
                    a3 = magic_sub(prmt(vh, 0x64646464u, 0x4341u), 0x64046404u);
                } else {
                    const int p = i >> 1;
                    const uint32_t wg = p ? u.z : u.x, wh = p ? u.w : u.y;
                    if ((i & 1) == 0) {
                        a0 = wg & 0x8E008E00u, a1 = wh & 0x8E008E00u;
                        a2 = (wg << 3) & 0x8E008E00u, a3 = (wh << 3) & 0x8E008E00u;
                    } else {
                        a0 = and_or(wg << 6, 0x0E000E00u, (wg << 2) & 0x80008000u), a1 = and_or(wh << 6, 0x0E000E00u, (wh << 2) & 0x80008000u);
                        a2 = and_or(wg << 9, 0x0E000E00u, (wg << 1) & 0x80008000u), a3 = and_or(wh << 9, 0x0E000E00u, (wh << 1) & 0x80008000u);
                    }
                }
                float c[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.f;
                    const uint2 b = load_b(xfrag, chunk0 + s, nt, NT, mst, g, t);
                    mma16816(c[nt], a0, a1, a2, a3, b.x, b.y);
                }
                scale_acc<NT>(acc, c, sg[s], sh[s]);
            }
        }
    }
}

template <int FMT, int NT>
__global__ void __launch_bounds__(512) gemv_t16_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int TB = kyb_tile_bytes(FMT);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kp = blockIdx.y;
    const int kb0 = kp * p.kbp, nblk = min(p.nb, kb0 + p.kbp) - kb0;
    const int mst = p.mst;

    // ---- shared memory carve-up
    const size_t xfrag_bytes = (size_t)p.kbp * 16 * NT * mst * 32;
    uint8_t* xfrag = smem;
    uint8_t* xaux = xfrag + xfrag_bytes;
    const size_t xaux_bytes = (size_t)p.kbp * xaux_bytes_per_block<FMT>(NT);
    const size_t warp_bytes = (size_t)p.stages * TB + SCL_BYTES + 8 * (size_t)p.stages + 8;
    uint8_t* wbase = xaux + xaux_bytes + (size_t)warp * ((warp_bytes + 15) & ~(size_t)15);
    uint8_t* ring = wbase;
    float* scl = reinterpret_cast<float*>(wbase + (size_t)p.stages * TB);
    uint64_t* bars = reinterpret_cast<uint64_t*>(wbase + (size_t)p.stages * TB + SCL_BYTES);

    const int rt = blockIdx.x * p.warps + warp;
    const bool active = rt < p.npad / 16 && nblk > 0;
    const uint8_t* src = p.t16 + ((size_t)rt * p.nb + kb0) * TB;

    // ---- start the weight stream before staging x: the copies run while the CTA prepares the activations
    if (lane == 0) {
        for (int s = 0; s < p.stages; ++s) mbar_init(&bars[s], 1);
        mbar_fence_init();
        if (active) {
            const int pre = min(p.stages, nblk);
            for (int s = 0; s < pre; ++s) {
                mbar_expect_tx(&bars[s], TB);
                bulk_g2s(ring + (size_t)s * TB, src + (size_t)s * TB, TB, &bars[s]);
            }
        }
    }

    // ---- stage activations of this k-part as B fragments: [chunk][nt][row < mst][lane t][4 halves permuted (0, 2, 1, 3)]
    {
        const int nchunk = nblk * 16;
        const int items = nchunk * NT * mst;
        for (int it = threadIdx.x; it < items; it += blockDim.x) {
            const int row = it % mst, nt = (it / mst) % NT, c = it / (mst * NT);
            const int m = nt * 8 + row;
            uint4 a = make_uint4(0, 0, 0, 0), b = make_uint4(0, 0, 0, 0);
            if (m < p.m) {
                const uint4* xp = reinterpret_cast<const uint4*>(p.x + (size_t)m * p.ldx + (size_t)kb0 * 256 + (size_t)c * 16);
                a = __ldg(xp), b = __ldg(xp + 1);
            }
            uint4 oa, ob;
            oa.x = prmt(a.x, a.y, 0x5410u), oa.y = prmt(a.x, a.y, 0x7632u), oa.z = prmt(a.z, a.w, 0x5410u), oa.w = prmt(a.z, a.w, 0x7632u);
            ob.x = prmt(b.x, b.y, 0x5410u), ob.y = prmt(b.x, b.y, 0x7632u), ob.z = prmt(b.z, b.w, 0x5410u), ob.w = prmt(b.z, b.w, 0x7632u);
            uint4* dst = reinterpret_cast<uint4*>(xfrag + ((size_t)(c * NT + nt) * mst + row) * 32);
            dst[0] = oa, dst[1] = ob;
        }
        if constexpr (FMT == KYB_FMT_Q4_K) {
            __syncthreads();
            // sums of x over each 32-input sub-block, split into fp16 hi + lo, laid out as m16n8k8 B fragments
            const int items2 = nblk * 8 * NT * 8;
            for (int it = threadIdx.x; it < items2; it += blockDim.x) {
                const int g_ = it & 7, nt = (it >> 3) % NT, j = (it / (8 * NT)) & 7, blk = it / (64 * NT);
                float sum = 0.f;
                if (g_ < mst) {
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const __half2* hp = reinterpret_cast<const __half2*>(xfrag + ((size_t)((blk * 16 + 2 * j + c) * NT + nt) * mst + g_) * 32);
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const float2 f = __half22float2(hp[q]);
                            sum += f.x + f.y;
                        }
                    }
                }
                const __half hi = __float2half_rn(sum);
                const __half lo = __float2half_rn(sum - __half2float(hi));
                __half* xa = reinterpret_cast<__half*>(xaux + (size_t)blk * 256 * NT);
                const int idx = (g_ * 4 + (j >> 1)) * 2 + (j & 1);
                xa[((0 * NT + nt) * 32) * 2 + idx] = hi;
                xa[((1 * NT + nt) * 32) * 2 + idx] = lo;
            }
        }
    }
    __syncthreads();
    if (!active) return;

    Acc<NT> acc;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc.v[nt][0] = acc.v[nt][1] = acc.v[nt][2] = acc.v[nt][3] = 0.f;

    bool alive = true;
    int bi = 0;
    for (; bi < nblk; ++bi) {
        const int st = bi % p.stages;
        const uint32_t parity = (uint32_t)(bi / p.stages) & 1u;
        const bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bars[st], parity));
        if (!ok) {
            alive = false;
            break;
        }
        const uint8_t* tile = ring + (size_t)st * TB;
        prep_scales<FMT>(tile, scl, lane);
        __syncwarp();
        consume_tile<FMT, NT>(tile, scl, xfrag, xaux, bi, mst, lane, acc);
        __syncwarp();
        if (lane == 0 && bi + p.stages < nblk) {
            mbar_expect_tx(&bars[st], TB);
            bulk_g2s(ring + (size_t)st * TB, src + (size_t)(bi + p.stages) * TB, TB, &bars[st]);
        }
    }
    if (!alive) {
        // record the failure, then give the copies still in flight a bounded chance to land before leaving
        if (lane == 0) atomicExch(p.status, KYB_DEV_TIMEOUT_GEMV);
        for (int b2 = bi + 1; b2 < min(nblk, bi + p.stages); ++b2) mbar_wait_bounded(&bars[b2 % p.stages], (uint32_t)(b2 / p.stages) & 1u, 1u << 16);
        return;
    }

    // ---- epilogue: lane (g, t) holds rows g, g + 8 x activation rows 2t, 2t + 1 of each column tile
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int nrow = rt * 16 + g + 8 * (i >> 1), m = nt * 8 + 2 * t + (i & 1);
            if (m >= p.m) continue;
            if (p.ksplit == 1) {
                if (nrow < p.n) p.y[(size_t)m * p.ldy + nrow] = sat_half(acc.v[nt][i] * p.gscale);
            } else {
                p.partial[((size_t)kp * p.m + m) * p.npad + nrow] = acc.v[nt][i];
            }
        }
    }
}

__global__ void gemv_finalize_kernel(const float* __restrict__ partial, int ksplit, int m, int n, int npad, float gscale, __half* __restrict__ y, int64_t ldy) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)m * n) return;
    const int row = (int)(i / n), col = (int)(i % n);
    float s = 0.f;
    for (int kp = 0; kp < ksplit; ++kp) s += partial[((size_t)kp * m + row) * npad + col];
    y[(size_t)row * ldy + col] = sat_half(s * gscale);
}

}  // namespace kyb

// ------------------------------------------------------------------------------------------------ host side
namespace {

struct GemvPlan {
    int nt, mst, warps, stages, kbp, ksplit;
    size_t smem;
};

int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return v && *v ? atoi(v) : dflt;
}

size_t plan_smem(int fmt, int nt, int mst, int kbp, int warps, int stages) {
    const size_t tb = kyb_tile_bytes(fmt);
    const size_t xfrag = (size_t)kbp * 16 * nt * mst * 32;
    const size_t xaux = fmt == KYB_FMT_Q4_K ? (size_t)kbp * 256 * nt : 0;
    const size_t wb = ((size_t)stages * tb + kyb::SCL_BYTES + 8 * (size_t)stages + 8 + 15) & ~(size_t)15;
    return xfrag + xaux + warps * wb;
}

// Picks warps per CTA, ring depth and the k split from a small cost model: whole waves of CTAs, >= 64 KB of bulk copies in
// flight per SM, split-k traffic counted. Environment overrides (KYB_GEMV_WARPS / _STAGES / _KSPLIT) exist for sweeps.
const void* gemv_kernel_ptr(int fmt, int nt) {
    static const void* tab[4][3] = {
        {(const void*)kyb::gemv_t16_kernel<KYB_FMT_Q4_K, 1>, (const void*)kyb::gemv_t16_kernel<KYB_FMT_Q4_K, 2>, (const void*)kyb::gemv_t16_kernel<KYB_FMT_Q4_K, 4>},
        {(const void*)kyb::gemv_t16_kernel<KYB_FMT_Q6_K, 1>, (const void*)kyb::gemv_t16_kernel<KYB_FMT_Q6_K, 2>, (const void*)kyb::gemv_t16_kernel<KYB_FMT_Q6_K, 4>},
        {(const void*)kyb::gemv_t16_kernel<KYB_FMT_Q3_K, 1>, (const void*)kyb::gemv_t16_kernel<KYB_FMT_Q3_K, 2>, (const void*)kyb::gemv_t16_kernel<KYB_FMT_Q3_K, 4>},
        {(const void*)kyb::gemv_t16_kernel<KYB_FMT_NVFP4, 1>, (const void*)kyb::gemv_t16_kernel<KYB_FMT_NVFP4, 2>, (const void*)kyb::gemv_t16_kernel<KYB_FMT_NVFP4, 4>}};
    return tab[fmt][nt == 1 ? 0 : nt == 2 ? 1 : 2];
}

// registers per thread of a kernel instantiation (cached; 128 = the launch bound, used when the query fails, e.g. without a device)
int gemv_kernel_regs(int fmt, int nt) {
    static int cache[4][3] = {{0}};
    int& c = cache[fmt][nt == 1 ? 0 : nt == 2 ? 1 : 2];
    if (!c) {
        cudaFuncAttributes a;
        c = cudaFuncGetAttributes(&a, gemv_kernel_ptr(fmt, nt)) == cudaSuccess && a.numRegs > 0 ? a.numRegs : 128;
        (void)cudaGetLastError();
    }
    return c;
}

GemvPlan make_plan(int fmt, int64_t n, int64_t k, int64_t m) {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        (void)cudaGetLastError();
    }
    GemvPlan best{};
    const int nt = m <= 8 ? 1 : m <= 16 ? 2 : 4;
    const int regs = (gemv_kernel_regs(fmt, nt) + 7) / 8 * 8;
    const int mst = m >= 8 ? 8 : m > 2 ? 4 : m > 1 ? 2 : 1;
    const int nb = (int)(k / 256), ntiles = (int)((n + 15) / 16);
    const double tb = kyb_tile_bytes(fmt), sm_bw = 6.8e12 / sms;          // bytes/s one SM can expect
    const size_t smem_cap = 227 * 1024, smem_sm = 228 * 1024;
    double best_t = 1e30;
    const int fw = env_int("KYB_GEMV_WARPS", 0), fs = env_int("KYB_GEMV_STAGES", 0), fk = env_int("KYB_GEMV_KSPLIT", 0);
    for (int ksplit = 1; ksplit <= nb; ++ksplit) {
        if (fk && ksplit != fk) continue;
        const int kbp = (nb + ksplit - 1) / ksplit;
        if ((nb + kbp - 1) / kbp != ksplit) continue;                      // skip splits that leave an empty part
        for (int warps = 1; warps <= 16; ++warps) {
            if (fw && warps != fw) continue;
            for (int stages = 2; stages <= 8; ++stages) {
                if (fs && stages != fs) continue;
                if (stages > kbp && stages > 2) continue;
                const size_t smem = plan_smem(fmt, nt, mst, kbp, warps, stages);
                if (smem > smem_cap) continue;
                int conc = (int)std::min<size_t>(smem_sm / (smem + 1024), (size_t)(64 / warps));
                conc = std::min(conc, std::min(16, 65536 / (regs * warps * 32)));
                if (conc < 1) continue;
                const int64_t ctas = (int64_t)((ntiles + warps - 1) / warps) * ksplit;
                const double waves = (double)((ctas + (int64_t)sms * conc - 1) / ((int64_t)sms * conc));
                const double cta_bytes = (double)warps * kbp * tb;
                const double inflight = (double)conc * warps * std::min(stages, kbp) * tb;
                const double bw_eff = sm_bw * std::min(1.0, inflight / 65536.0);
                double tsec = waves * (cta_bytes * conc / bw_eff + 1.0e-6 / conc);
                if (ksplit > 1) tsec += 2.0 * ksplit * m * (double)n * 4.0 / 6.8e12 + 1.5e-6;
                tsec += 1e-9 * stages;                                      // tie-break: shallower ring
                if (tsec < best_t) best_t = tsec, best = GemvPlan{nt, mst, warps, stages, kbp, ksplit, smem};
            }
        }
    }
    return best;
}

template <int FMT>
int launch_gemv(const kyb::GemvParams& p, const GemvPlan& pl, cudaStream_t st) {
    dim3 grid((unsigned)((p.npad / 16 + pl.warps - 1) / pl.warps), (unsigned)pl.ksplit), block((unsigned)pl.warps * 32);
    auto go = [&](auto kern) -> int {
        // opt in to large dynamic shared memory once per device and kernel instantiation (the attribute is per device)
        static std::atomic<unsigned> configured{0};
        int dev = 0;
        KYB_CUDA(cudaGetDevice(&dev));
        if (!(configured.load() & (1u << (dev & 31)))) {
            KYB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(227 * 1024)));
            configured.fetch_or(1u << (dev & 31));
        }
        kern<<<grid, block, pl.smem, st>>>(p);
        return kyb_launch_check("gemv_t16");
    };
    switch (pl.nt) {
        case 1: return go(kyb::gemv_t16_kernel<FMT, 1>);
        case 2: return go(kyb::gemv_t16_kernel<FMT, 2>);
        default: return go(kyb::gemv_t16_kernel<FMT, 4>);
    }
}

}  // namespace

extern "C" size_t kyb_gemv_workspace_bytes(int fmt, int64_t n, int64_t k, int64_t m) {
    if (fmt < 0 || fmt > 3 || n <= 0 || k <= 0 || k % 256 || m <= 0 || m > 32) return 0;
    const GemvPlan pl = make_plan(fmt, n, k, m);
    return pl.ksplit > 1 ? (size_t)pl.ksplit * (size_t)m * (size_t)((n + 15) / 16 * 16) * sizeof(float) : 0;
}

extern "C" int kyb_gemv_t16(int fmt, const void* t16, int64_t n, int64_t k, const void* x, int64_t m, int64_t ldx, float gscale, void* y, int64_t ldy,
                            void* workspace, size_t workspace_bytes, void* stream) {
    KYB_REQUIRE(fmt >= 0 && fmt <= 3, "unknown weight format %d", fmt);
    KYB_REQUIRE(n > 0 && k > 0 && k % 256 == 0, "n=%lld k=%lld: k must be a positive multiple of 256", (long long)n, (long long)k);
    KYB_REQUIRE(m >= 1 && m <= 32, "m=%lld: this entry point serves 1..32 activation rows", (long long)m);
    KYB_REQUIRE(t16 && x && y, "null pointer");
    KYB_REQUIRE(((uintptr_t)t16 & 15) == 0 && ((uintptr_t)x & 15) == 0, "t16 and x must be 16-byte aligned");
    KYB_REQUIRE(ldx >= k && ldx % 8 == 0, "ldx=%lld must be >= k and a multiple of 8", (long long)ldx);
    KYB_REQUIRE(ldy >= n, "ldy=%lld must be >= n", (long long)ldy);
    KYB_REQUIRE(n <= (int64_t)1 << 30 && k <= (int64_t)1 << 24, "matrix too large for 32-bit tile indices");
    const GemvPlan pl = make_plan(fmt, n, k, m);
    KYB_REQUIRE(pl.warps > 0, "no launch configuration fits shared memory for k=%lld m=%lld", (long long)k, (long long)m);
    const int npad = (int)((n + 15) / 16 * 16);
    const size_t need = pl.ksplit > 1 ? (size_t)pl.ksplit * (size_t)m * (size_t)npad * sizeof(float) : 0;
    if (need && (!workspace || workspace_bytes < need)) {
        kyb_set_error("gemv needs %zu bytes of workspace, got %zu", need, workspace ? workspace_bytes : (size_t)0);
        return KYB_EWORKSPACE;
    }
    unsigned int* status = kyb_device_status_word();
    KYB_REQUIRE(status, "could not set up the device status word");
    kyb::GemvParams p;
    p.t16 = (const uint8_t*)t16, p.x = (const __half*)x, p.y = (__half*)y, p.partial = (float*)workspace, p.status = status;
    p.ldx = ldx, p.ldy = ldy, p.n = (int)n, p.npad = npad, p.nb = (int)(k / 256), p.m = (int)m, p.mst = pl.mst;
    p.kbp = pl.kbp, p.ksplit = pl.ksplit, p.warps = pl.warps, p.stages = pl.stages, p.gscale = gscale;
    cudaStream_t st = (cudaStream_t)stream;
    int rc;
    switch (fmt) {
        case KYB_FMT_Q4_K: rc = launch_gemv<KYB_FMT_Q4_K>(p, pl, st); break;
        case KYB_FMT_Q6_K: rc = launch_gemv<KYB_FMT_Q6_K>(p, pl, st); break;
        case KYB_FMT_Q3_K: rc = launch_gemv<KYB_FMT_Q3_K>(p, pl, st); break;
        default: rc = launch_gemv<KYB_FMT_NVFP4>(p, pl, st); break;
    }
    if (rc) return rc;
    if (pl.ksplit > 1) {
        const int64_t tot = m * n;
        kyb::gemv_finalize_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, st>>>((const float*)workspace, pl.ksplit, (int)m, (int)n, npad, gscale, (__half*)y, ldy);
        return kyb_launch_check("gemv_finalize");
    }
    return KYB_OK;
}
