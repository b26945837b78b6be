// Prefill GEMM with the dequantisation fused into the operand producer: D[m, n] = sat_f16(gscale * sum_k A[m, k] * W[n, k]), W read as T16 tiles
// (every format of the library) and never written to HBM as fp16. Replaces the two-step large-row path of kyojin_mlx/foreign_linear.py:710 / :737
// (`x2 @ self.dequant().T`) and, in grouped form, the sorted grouped product of kyojin_mlx/foreign_kqgmm.py:225-239 (`gmm`).
//
// One persistent CTA per SM, 22 warps:
//   warp 0      TMA: activation tiles (128 rows x 64 inputs, 128-byte swizzle) into the stage ring
//   warp 1      tcgen05.mma issuer (UMMA 128 x 256 x 16, kind::f16, fp32 accumulators in tensor memory), stages handed back by tcgen05.commit
//   warps 2-5   epilogue: tcgen05.ld, output scale, saturating fp16 stores
//   warps 6-21  decoders: warp w owns the 16-row T16 row tile w of the CTA's 256 weight rows. It keeps one T16 tile (256 inputs) in registers (the next one
//               is already in flight), and for each 64-input quarter unpacks the codes with LOP3 / PRMT into fp16 pairs, applies the block scales with
//               half2 arithmetic (scale and min rounded to fp16, then one fma per pair: the rounding points of the reference's few-row kernels,
//               kyojin_mlx/foreign_metal.py:1357-1358, :1382-1383) and writes the pairs into the stage's B tile in the swizzled K-major layout the UMMA
//               descriptor expects, followed by a proxy fence and one mbarrier arrival per warp.
// A work item is a 256-row block of W times one or two 128-row blocks of A (msub): with two, a decoded weight serves 256 activation rows, which halves the
// decode work per flop; with one, the two tensor-memory accumulators alternate and the epilogue overlaps the next item's MMAs (grouped form: an expert's
// segment is cut into 128-row tiles). Every mbarrier wait is bounded; a wait that gives up sets the device status word and the CTA drains.
#include <algorithm>
#include <cstring>
#include <mutex>

#include "t16_decode.cuh"
#include "tc_common.cuh"

namespace kyb {

constexpr int KQ_BN = 256, KQ_BK = 64, KQ_DW = 16, KQ_THREADS = (6 + KQ_DW) * 32;
constexpr uint32_t KQ_A_SUB = 128 * KQ_BK * 2, KQ_B_BYTES = KQ_BN * KQ_BK * 2;
constexpr int KQ_TORD = 2048;                          // grouped form: tile order table in shared memory (u16 entries)
constexpr uint32_t KQ_SCR = 1280;                       // per decoder warp: block scales of one T16 tile as half2 pairs
constexpr uint32_t KQ_STG = KYB_STG_BYTES;              // per epilogue warp: 32 rows x 32 fp16 columns staged for a tiled bulk store
using KqOutMaps = KybOutMaps;                           // dense form: the [m, col0 + n] fp16 output matrix of every receiving rank

struct KqParams {
    const uint8_t* t16;
    __half* d[8];               // output matrix on every rank that receives the tiles (one entry without sharding), already offset to this rank's first column
    int nout;
    int64_t ldd;
    int m, n, k, nb;            // rows of A, rows of one W matrix, inputs, 256-input blocks
    int rt_total;               // 16-row tiles in the whole T16 buffer (row tiles past it are clamped; their columns are never stored)
    float gscale;
    unsigned int* status;
    const uint32_t* tb;         // grouped form: first (128 msub)-row tile of every expert (E + 1 entries), else null
    const uint32_t* off;        // grouped form: first sorted row of every expert (E + 1 entries)
    const uint32_t* row_map;    // optional: output row of every sorted row
    const float* gs;            // optional: per-expert output scale
    int experts;
    int tiles_m, tiles_n;
    int msub, stages;
    int tma_out, col0;          // dense form: the epilogue stores through the tensor maps (bulk tiled stores), at column col0 + n0
    int wide;                   // ... in 32 x 64 boxes (4 KB of staging per epilogue warp) instead of 32 x 32: used when the tiles also go to other GPUs
    // gated pair (grouped form): an item's 256 weight rows are 128 rows of the gate stack (t16) and the same 128 rows of the up stack (t16b); the epilogue writes
    // fp16(silu(a) * b) of the two fp16-rounded products, 128 output columns per item (kyojin_mlx/foreign_kqgmm.py:293-314 `mlp`: gmm, gmm, silu_perm in one launch)
    // split-k (dense form, one destination): the k-blocks are cut into ksplit equal ranges, an item is (tile, range) and writes its fp32 accumulator to
    // part [range][m][ldp] instead of d; gemm_kq_reduce_kernel adds the ranges in k order, scales, saturates and stores d
    int ksplit, mpad;           // mpad: rows of a range in part (m rounded up to whole items)
    float* part;
    int64_t ldp;
    const uint8_t* t16b;
    const float* gsb;           // per-expert output scale of the up stack (or null)
    int glu;
    float limit;                // > 0: a = min(a, limit), b = clamp(b, -limit, limit) as the activation kernel does
};

struct KqItem {
    int m0, m_end, n0, b_rt0, nsub;
    int tb0, ntb, sp;           // first 256-input block, number of blocks and index of the item's k-range (the whole of k without split-k)
    float gscale, gscale_b;
    bool valid;
};

__device__ __forceinline__ KqItem kq_item(const KqParams& p, int t, const uint16_t* tord = nullptr) {
    KqItem it;
    it.valid = true, it.gscale = p.gscale, it.gscale_b = p.gscale, it.m_end = p.m;
    it.tb0 = 0, it.ntb = p.nb, it.sp = 0;
    if (!p.tb) {
        if (p.ksplit > 1) {                                                             // tiles fastest, k-ranges slowest
            const int tiles = p.tiles_m * p.tiles_n;
            it.sp = t / tiles, t -= it.sp * tiles;
            it.ntb = p.nb / p.ksplit, it.tb0 = it.sp * it.ntb;
        }
        const int tn = t / p.tiles_m, tm = t - tn * p.tiles_m;                         // m fastest: CTAs running together share the weight rows
        it.n0 = tn * KQ_BN, it.m0 = tm * 128 * p.msub, it.b_rt0 = it.n0 >> 4;
        it.nsub = min(p.msub, (p.m - it.m0 + 127) >> 7);
        return it;
    }
    int tm = t / p.tiles_n;
    const int tn = t - tm * p.tiles_n;                                                   // n fastest: CTAs running together share the activation rows
    it.n0 = tn * (p.glu ? KQ_BN / 2 : KQ_BN);
    if ((uint32_t)tm >= p.tb[p.experts]) {
        it.valid = false;
        return it;
    }
    if (tord) tm = (int)tord[tm];                                                        // two-block tiles first (see the kernel's prologue)
    int lo = 0, hi = p.experts;                                                          // largest e with tb[e] <= tm (empty experts repeat a value)
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (p.tb[mid] <= (uint32_t)tm) lo = mid; else hi = mid;
    }
    it.m0 = (int)(p.off[lo] + ((uint32_t)tm - p.tb[lo]) * (uint32_t)(128 * p.msub));
    it.m_end = (int)p.off[lo + 1];
    it.nsub = min(p.msub, (it.m_end - it.m0 + 127) >> 7);                                // a segment tail of up to 128 rows runs one block
    it.b_rt0 = (lo * p.n + it.n0) >> 4;
    if (p.gs) it.gscale = p.gs[lo];
    if (p.gsb) it.gscale_b = p.gsb[lo];
    return it;
}

// ------------------------------------------------------------------------------------------------ decoder: tile registers, scales, quarters
__device__ __forceinline__ uint4 ldg128s(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg64s(const uint8_t* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg32s(const uint8_t* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg16s(const uint8_t* p) {
    unsigned short v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ void sts64(uint32_t a, uint32_t x, uint32_t y) { asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(a), "r"(x), "r"(y) : "memory"); }
__device__ __forceinline__ void sts128(uint32_t a, uint4 v) { asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory"); }

__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
    __half2 r = __hsub2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t h2_mul(uint32_t a, uint32_t b) {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
    __half2 r = __hfma2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b), *reinterpret_cast<__half2*>(&c));
    return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t h2_splat(float v) {
    __half2 r = __half2half2(sat_half(v));
    return *reinterpret_cast<uint32_t*>(&r);
}

// What one lane holds of a T16 tile: its 16-byte units of the code planes (the lane's MMA-fragment bytes, see kyojin_mac_b200/layout.py) and the scale bytes
// of row lane / 2 (half lane % 2) for the scale preparation.
template <int FMT>
struct KqTile {
    uint4 q[FMT == KYB_FMT_Q6_K ? 6 : FMT == KYB_FMT_Q3_K ? 3 : FMT == KYB_FMT_Q5_K ? 5 : FMT == KYB_FMT_Q8_0 ? 8 : FMT == KYB_FMT_Q2_K ? 2 : 4];
    uint4 sc;
    uint32_t d16;
};

template <int FMT>
__device__ __forceinline__ void kq_load(const uint8_t* tile, int lane, KqTile<FMT>& tr) {
    const int r = lane >> 1, hf = lane & 1;
    if constexpr (FMT == KYB_FMT_Q4_K) {
#pragma unroll
        for (int G = 0; G < 4; ++G) tr.q[G] = ldg128s(tile + (G * 32 + lane) * 16);
        tr.sc = ldg128s(tile + 2048 + r * 16);
        tr.d16 = 0;
    } else if constexpr (FMT == KYB_FMT_Q5_K) {
#pragma unroll
        for (int P = 0; P < 4; ++P) tr.q[P] = ldg128s(tile + (P * 32 + lane) * 16);
        tr.q[4] = ldg128s(tile + 2048 + lane * 16);                                           // the fifth bits of all four quarters
        tr.sc = ldg128s(tile + 2560 + r * 16);
        tr.d16 = 0;
    } else if constexpr (FMT == KYB_FMT_Q8_0) {
#pragma unroll
        for (int P = 0; P < 8; ++P) tr.q[P] = ldg128s(tile + (P * 32 + lane) * 16);
        tr.sc = ldg128s(tile + 4096 + r * 16);                                                // the row's eight fp16 d
        tr.d16 = 0;
    } else if constexpr (FMT == KYB_FMT_Q2_K) {
        tr.q[0] = ldg128s(tile + lane * 16);
        tr.q[1] = ldg128s(tile + (32 + lane) * 16);
        tr.sc = ldg128s(tile + 1024 + r * 16);                                                // the row's 16 scale | min << 4 bytes
        tr.d16 = ldg32s(tile + 1280 + r * 4);                                                 // d | dmin << 16
    } else if constexpr (FMT == KYB_FMT_IQ4_XS) {
#pragma unroll
        for (int P = 0; P < 4; ++P) tr.q[P] = ldg128s(tile + (P * 32 + lane) * 16);
        const uint2 mw = ldg64s(tile + 2048 + r * 8);                                         // d | scales_h << 16, four scales_l bytes
        tr.sc = make_uint4(mw.x, mw.y, 0, 0);
        tr.d16 = 0;
    } else if constexpr (FMT == KYB_FMT_Q6_K) {
#pragma unroll
        for (int P = 0; P < 4; ++P) tr.q[P] = ldg128s(tile + (P * 32 + lane) * 16);
        tr.q[4] = ldg128s(tile + 2048 + lane * 16);
        tr.q[5] = ldg128s(tile + 2048 + (32 + lane) * 16);
        const uint2 s = ldg64s(tile + 3072 + r * 16 + 8 * hf);
        tr.sc = make_uint4(s.x, s.y, 0, 0);
        tr.d16 = ldg16s(tile + 3328 + r * 2);
    } else if constexpr (FMT == KYB_FMT_Q3_K) {
        tr.q[0] = ldg128s(tile + lane * 16);
        tr.q[1] = ldg128s(tile + (32 + lane) * 16);
        tr.q[2] = ldg128s(tile + 1024 + lane * 16);
        const uint8_t* sp = tile + 1536 + r * 12;
        tr.sc = make_uint4(ldg32s(sp), ldg32s(sp + 4), ldg32s(sp + 8), 0);
        tr.d16 = ldg16s(tile + 1728 + r * 2);
    } else {
#pragma unroll
        for (int P = 0; P < 4; ++P) tr.q[P] = ldg128s(tile + (P * 32 + lane) * 16);
        const uint2 s = ldg64s(tile + 2048 + r * 16 + 8 * hf);
        tr.sc = make_uint4(s.x, s.y, 0, 0);
        tr.d16 = 0;
    }
}

// Block scales of the tile as half2 pairs (value, value) in the warp's scratch. Q4_K: S[row][8] at row * 32, Z[row][8] at 512 + row * 32 (scale and minus min of
// the eight 32-input sub-blocks); the others: S[row][16] at row * 80 (one scale per 16 inputs; the 80-byte pitch keeps the 16-byte reads of 8 rows on distinct banks).
// (lo, hi) fp16 pair -> the two (v, v) pairs, clamped to the finite fp16 range (an overflowing block scale must not turn into inf * 0)
__device__ __forceinline__ uint32_t h2_clamp(uint32_t a) {
    __half2 v = *reinterpret_cast<__half2*>(&a);
    const uint32_t hi_bits = 0x7BFF7BFFu, lo_bits = 0xFBFFFBFFu;
    v = __hmax2(__hmin2(v, *reinterpret_cast<const __half2*>(&hi_bits)), *reinterpret_cast<const __half2*>(&lo_bits));
    return *reinterpret_cast<uint32_t*>(&v);
}
// four byte codes c (unsigned, as (1024 + c) - bias in fp16, exact) times the fp16 pair d2 -> four (v, v) pairs; fp16(d * code) is the single rounding of the
// exact product, the same value as the float32 product rounded to fp16
__device__ __forceinline__ uint4 kq_scale4(uint32_t codes, uint32_t bias2, uint32_t d2) {
    const uint32_t a = h2_clamp(h2_mul(h2_sub(prmt(codes, 0x64646464u, 0x4140u), bias2), d2));
    const uint32_t b = h2_clamp(h2_mul(h2_sub(prmt(codes, 0x64646464u, 0x4342u), bias2), d2));
    return make_uint4(prmt(a, 0u, 0x1010u), prmt(a, 0u, 0x3232u), prmt(b, 0u, 0x1010u), prmt(b, 0u, 0x3232u));
}

// Block scales of the tile as half2 pairs (value, value) in the warp's scratch. Q4_K / Q5_K: (S, Z)[row][8] at row * 80 (scale and minus min of the eight
// 32-input sub-blocks, interleaved: one 16-byte read gives both of the two sub-blocks of a quarter); Q8_0 / IQ4_XS: S[row][8] at row * 48; the others: S[row][16]
// at row * 80 (one scale per 16 inputs). With the 80- and 48-byte pitches the reads of rows g = 0 .. 7 fall on distinct banks: a warp's read costs the minimum
// number of shared-memory wavefronts (a 32-byte pitch puts rows g and g + 4 on the same banks and doubles them).
template <int FMT>
__device__ __forceinline__ void kq_prep_scales(const KqTile<FMT>& tr, uint32_t scr, int lane) {
    const int r = lane >> 1, hf = lane & 1;
    if constexpr (FMT == KYB_FMT_Q2_K) {
        // one scale and one minimum per 16 inputs: word (fp16(d sc), fp16(-dmin mn)) per slice at row * 80 + 4 * slice (lane half hf covers slices 8 hf .. 8 hf + 7)
        const uint32_t d2 = prmt(tr.d16, 0u, 0x1010u), dm2 = prmt(tr.d16, 0u, 0x3232u) ^ 0x80008000u;
        const uint32_t w0 = hf ? tr.sc.z : tr.sc.x, w1 = hf ? tr.sc.w : tr.sc.y;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const uint32_t w = q ? w1 : w0;
            const uint32_t sl = w & 0x0F0F0F0Fu, ml = (w >> 4) & 0x0F0F0F0Fu;
            const uint32_t sa = h2_clamp(h2_mul(h2_sub(prmt(sl, 0x64646464u, 0x4140u), 0x64006400u), d2)), sb = h2_clamp(h2_mul(h2_sub(prmt(sl, 0x64646464u, 0x4342u), 0x64006400u), d2));
            const uint32_t za = h2_clamp(h2_mul(h2_sub(prmt(ml, 0x64646464u, 0x4140u), 0x64006400u), dm2)), zb = h2_clamp(h2_mul(h2_sub(prmt(ml, 0x64646464u, 0x4342u), 0x64006400u), dm2));
            sts128(scr + r * 80 + 32 * hf + 16 * q, make_uint4(prmt(sa, za, 0x5410u), prmt(sa, za, 0x7632u), prmt(sb, zb, 0x5410u), prmt(sb, zb, 0x7632u)));
        }
    } else if constexpr (FMT == KYB_FMT_IQ4_XS) {
        // 6-bit scales of sub-blocks 4 hf .. 4 hf + 3 (4 low bits from scales_l, 2 high bits from scales_h), minus 32, times d: S[row][8] as (v, v) pairs at row * 32
        const uint32_t sh = tr.sc.x >> (16 + 8 * hf), sl = tr.sc.y >> (16 * hf);
        const uint32_t lsw = ((sl & 15u) | ((sh & 3u) << 4)) | ((((sl >> 4) & 15u) | (((sh >> 2) & 3u) << 4)) << 8) | ((((sl >> 8) & 15u) | (((sh >> 4) & 3u) << 4)) << 16) |
                             ((((sl >> 12) & 15u) | (((sh >> 6) & 3u) << 4)) << 24);
        sts128(scr + r * 48 + 16 * hf, kq_scale4(lsw, 0x64206420u, prmt(tr.sc.x, 0u, 0x1010u)));
    } else if constexpr (FMT == KYB_FMT_Q8_0) {
        // one fp16 d per 32 inputs: S[row][8] as (d, d) pairs at row * 32 (lane half hf covers blocks 4 hf .. 4 hf + 3)
        const uint32_t w0 = hf ? tr.sc.z : tr.sc.x, w1 = hf ? tr.sc.w : tr.sc.y;
        sts128(scr + r * 48 + 16 * hf, make_uint4(h2_clamp(prmt(w0, 0u, 0x1010u)), h2_clamp(prmt(w0, 0u, 0x3232u)), h2_clamp(prmt(w1, 0u, 0x1010u)), h2_clamp(prmt(w1, 0u, 0x3232u))));
    } else if constexpr (FMT == KYB_FMT_Q4_K || FMT == KYB_FMT_Q5_K) {
        const uint4 mt = tr.sc;
        const uint32_t scw = ((hf ? mt.w : mt.y) & (hf ? 0x0f0f0f0fu : 0x3f3f3f3fu)) | ((mt.y >> 2) & (hf ? 0x30303030u : 0u));
        const uint32_t mnw = ((hf ? mt.w >> 4 : mt.z) & (hf ? 0x0f0f0f0fu : 0x3f3f3f3fu)) | ((mt.z >> 2) & (hf ? 0x30303030u : 0u));
        const uint32_t d2 = prmt(mt.x, 0u, 0x1010u), dm2 = prmt(mt.x, 0u, 0x3232u) ^ 0x80008000u;           // (d, d) and (-dmin, -dmin)
        const uint4 sv = kq_scale4(scw, 0x64006400u, d2), zv = kq_scale4(mnw, 0x64006400u, dm2);
        sts128(scr + r * 80 + 32 * hf, make_uint4(sv.x, zv.x, sv.y, zv.y));
        sts128(scr + r * 80 + 32 * hf + 16, make_uint4(sv.z, zv.z, sv.w, zv.w));
    } else if constexpr (FMT == KYB_FMT_Q6_K) {
        const uint32_t d2 = prmt(tr.d16, 0u, 0x1010u);
        // int8 scale + 128 as an unsigned byte, bias 1024 + 128
        sts128(scr + r * 80 + 32 * hf, kq_scale4(tr.sc.x ^ 0x80808080u, 0x64806480u, d2));
        sts128(scr + r * 80 + 32 * hf + 16, kq_scale4(tr.sc.y ^ 0x80808080u, 0x64806480u, d2));
    } else if constexpr (FMT == KYB_FMT_Q3_K) {
        const uint32_t w0 = tr.sc.x, w1 = tr.sc.y, w2 = tr.sc.z;
        const uint32_t ga = hf ? (((w0 >> 4) & 0x0f0f0f0fu) | (w2 & 0x30303030u)) : ((w0 & 0x0f0f0f0fu) | ((w2 << 4) & 0x30303030u));
        const uint32_t gb = hf ? (((w1 >> 4) & 0x0f0f0f0fu) | ((w2 >> 2) & 0x30303030u)) : ((w1 & 0x0f0f0f0fu) | ((w2 << 2) & 0x30303030u));
        const uint32_t d2 = prmt(tr.d16, 0u, 0x1010u);
        sts128(scr + r * 80 + 32 * hf, kq_scale4(ga, 0x64206420u, d2));                                     // 6-bit scale - 32
        sts128(scr + r * 80 + 32 * hf + 16, kq_scale4(gb, 0x64206420u, d2));
    } else {
        // e4m3 magnitude (7 bits) << 7 is the fp16 of value * 2^-8; code 0x7F decodes to 0
        auto four = [](uint32_t w) -> uint4 {
            w &= 0x7f7f7f7fu;
            const uint32_t is7f = ((w + 0x01010101u) & 0x80808080u) >> 7;                                    // 1 in every byte that is 0x7F
            w ^= is7f * 0x7fu;
            const uint32_t a = h2_mul(prmt(w, 0u, 0x4140u) << 7, 0x5C005C00u), b = h2_mul(prmt(w, 0u, 0x4342u) << 7, 0x5C005C00u);   // * 2^8, exact
            return make_uint4(prmt(a, 0u, 0x1010u), prmt(a, 0u, 0x3232u), prmt(b, 0u, 0x1010u), prmt(b, 0u, 0x3232u));
        };
        sts128(scr + r * 80 + 32 * hf, four(tr.sc.x));
        sts128(scr + r * 80 + 32 * hf + 16, four(tr.sc.y));
    }
}

// Quarter P (inputs [64 P, 64 P + 64)) of the tile: this lane's fp16 weights of rows g (h = 0) and g + 8 (h = 1), four consecutive inputs of every 16-input slice i
// as the two registers r[4 i + 2 h], r[4 i + 2 h + 1].
template <int FMT, int P>
__device__ __forceinline__ void kq_compute_quarter(const KqTile<FMT>& tr, uint32_t scr, int lane, uint32_t (&r)[16]) {
    const int g = lane >> 2;
    if constexpr (FMT == KYB_FMT_Q4_K) {
        const uint4 u = tr.q[P];
        const uint4 sg = lds128(scr + g * 80 + 16 * P), sh = lds128(scr + (g + 8) * 80 + 16 * P);   // (scale, minus min) of sub-blocks 2 P and 2 P + 1
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t w = h ? (c ? u.w : u.y) : (c ? u.z : u.x);
                const uint32_t s_lo = h ? sh.x : sg.x, s_hi = h ? sh.z : sg.z, z_lo = h ? sh.y : sg.y, z_hi = h ? sh.w : sg.w;
                const uint32_t p01 = prmt(w, 0u, 0x4140u), p23 = prmt(w, 0u, 0x4342u);       // bytes (b0, 0, b1, 0), (b2, 0, b3, 0)
                // low nibbles: 1024 + q, minus 1024; high nibbles: (1024 + 16 q) / 16 - 64; both exact
                const uint32_t l01 = h2_sub(and_or(p01, 0x000F000Fu, 0x64006400u), 0x64006400u), l23 = h2_sub(and_or(p23, 0x000F000Fu, 0x64006400u), 0x64006400u);
                const uint32_t h01 = h2_fma(and_or(p01, 0x00F000F0u, 0x64006400u), 0x2C002C00u, 0xD400D400u);
                const uint32_t h23 = h2_fma(and_or(p23, 0x00F000F0u, 0x64006400u), 0x2C002C00u, 0xD400D400u);
                r[4 * c + 2 * h] = h2_fma(l01, s_lo, z_lo), r[4 * c + 2 * h + 1] = h2_fma(l23, s_lo, z_lo);
                r[4 * (2 + c) + 2 * h] = h2_fma(h01, s_hi, z_hi), r[4 * (2 + c) + 2 * h + 1] = h2_fma(h23, s_hi, z_hi);
            }
        }
    } else if constexpr (FMT == KYB_FMT_Q5_K) {
        const uint4 u = tr.q[P], hb = tr.q[4];
        const uint4 sg = lds128(scr + g * 80 + 16 * P), sh = lds128(scr + (g + 8) * 80 + 16 * P);   // (scale, minus min) of sub-blocks 2 P and 2 P + 1
#pragma unroll
        for (int i = 0; i < 4; ++i) {                                                    // slice s = 4 P + i, sub-block 2 P + i / 2
            const int p = i >> 1, i8 = 4 * (P & 1) + i;                                      // fifth bit of slice s: bit s & 7 of word s >> 3
            uint32_t wg = p ? u.z : u.x, wh = p ? u.w : u.y;
            if (i & 1) wg >>= 4, wh >>= 4;
            uint32_t bg = (P & 2) ? hb.z : hb.x, bh = (P & 2) ? hb.w : hb.y;
            if (i8 < 4) bg <<= (4 - i8), bh <<= (4 - i8);
            else bg >>= (i8 - 4), bh >>= (i8 - 4);
            const uint32_t vg = and_or(wg, 0x0F0F0F0Fu, bg & 0x10101010u), vh = and_or(wh, 0x0F0F0F0Fu, bh & 0x10101010u);
            // bytes -> fp16 (1024 + v) - 1024 = v, exact; then one fma per pair with the fp16 scale and minus min of the sub-block
            const uint32_t sgi = p ? sg.z : sg.x, zgi = p ? sg.w : sg.y, shi = p ? sh.z : sh.x, zhi = p ? sh.w : sh.y;
            r[4 * i] = h2_fma(h2_sub(prmt(vg, 0x64646464u, 0x4140u), 0x64006400u), sgi, zgi);
            r[4 * i + 1] = h2_fma(h2_sub(prmt(vg, 0x64646464u, 0x4342u), 0x64006400u), sgi, zgi);
            r[4 * i + 2] = h2_fma(h2_sub(prmt(vh, 0x64646464u, 0x4140u), 0x64006400u), shi, zhi);
            r[4 * i + 3] = h2_fma(h2_sub(prmt(vh, 0x64646464u, 0x4342u), 0x64006400u), shi, zhi);
        }
    } else if constexpr (FMT == KYB_FMT_Q2_K) {
        const uint4 u = tr.q[P >> 1];
        const uint4 sg4 = lds128(scr + g * 80 + 16 * P), sh4 = lds128(scr + (g + 8) * 80 + 16 * P);
        const uint32_t sg[4] = {sg4.x, sg4.y, sg4.z, sg4.w}, sh[4] = {sh4.x, sh4.y, sh4.z, sh4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {                                                    // slice 4 P + i: codes at bits 2 i of word (P & 1)
            const uint32_t vg = (((P & 1) ? u.z : u.x) >> (2 * i)) & 0x03030303u, vh = (((P & 1) ? u.w : u.y) >> (2 * i)) & 0x03030303u;
            const uint32_t Sg = prmt(sg[i], 0u, 0x1010u), Zg = prmt(sg[i], 0u, 0x3232u), Sh = prmt(sh[i], 0u, 0x1010u), Zh = prmt(sh[i], 0u, 0x3232u);
            r[4 * i] = h2_fma(h2_sub(prmt(vg, 0x64646464u, 0x4140u), 0x64006400u), Sg, Zg);
            r[4 * i + 1] = h2_fma(h2_sub(prmt(vg, 0x64646464u, 0x4342u), 0x64006400u), Sg, Zg);
            r[4 * i + 2] = h2_fma(h2_sub(prmt(vh, 0x64646464u, 0x4140u), 0x64006400u), Sh, Zh);
            r[4 * i + 3] = h2_fma(h2_sub(prmt(vh, 0x64646464u, 0x4342u), 0x64006400u), Sh, Zh);
        }
    } else if constexpr (FMT == KYB_FMT_IQ4_XS) {
        const uint4 u = tr.q[P];
        const uint2 sg = lds64(scr + g * 48 + 8 * P), sh = lds64(scr + (g + 8) * 48 + 8 * P);
        auto grid4 = [](uint32_t idx) -> uint32_t {                                      // four 4-bit codes (one per byte) -> their grid values + 128
            const uint32_t x = idx & 0x07070707u, y = x | (x >> 4);
            const uint32_t sel = prmt(y, 0u, 0x4420u);
            const uint32_t lo = prmt(0xBFAD9881u, 0xF6EADDCFu, sel), hi = prmt(0x26190D01u, 0x71594535u, sel);
            const uint32_t m = ((idx >> 3) & 0x01010101u) * 0xFFu;
            return ((lo & ~m) | (hi & m)) ^ 0x80808080u;
        };
#pragma unroll
        for (int i = 0; i < 4; ++i) {                                                    // slice 4 P + i, sub-block 2 P + i / 2
            const int p = i >> 1;
            uint32_t wg = p ? u.z : u.x, wh = p ? u.w : u.y;
            if (i & 1) wg >>= 4, wh >>= 4;
            const uint32_t vg = grid4(wg & 0x0F0F0F0Fu), vh = grid4(wh & 0x0F0F0F0Fu);
            const uint32_t sgi = p ? sg.y : sg.x, shi = p ? sh.y : sh.x;
            r[4 * i] = h2_mul(h2_sub(prmt(vg, 0x64646464u, 0x4140u), 0x64806480u), sgi);
            r[4 * i + 1] = h2_mul(h2_sub(prmt(vg, 0x64646464u, 0x4342u), 0x64806480u), sgi);
            r[4 * i + 2] = h2_mul(h2_sub(prmt(vh, 0x64646464u, 0x4140u), 0x64806480u), shi);
            r[4 * i + 3] = h2_mul(h2_sub(prmt(vh, 0x64646464u, 0x4342u), 0x64806480u), shi);
        }
    } else if constexpr (FMT == KYB_FMT_Q8_0) {
        const uint2 sg = lds64(scr + g * 48 + 8 * P), sh = lds64(scr + (g + 8) * 48 + 8 * P);
#pragma unroll
        for (int i = 0; i < 4; ++i) {                                                    // slice 4 P + i = half i & 1 of unit 2 P + i / 2 (one 32-input block)
            const uint4 u = tr.q[2 * P + (i >> 1)];
            const uint32_t vg = ((i & 1) ? u.z : u.x) ^ 0x80808080u, vh = ((i & 1) ? u.w : u.y) ^ 0x80808080u;   // int8 -> value + 128
            const uint32_t sgi = (i >> 1) ? sg.y : sg.x, shi = (i >> 1) ? sh.y : sh.x;
            // bytes -> fp16 (1024 + v + 128) - 1152 = v, exact
            r[4 * i] = h2_mul(h2_sub(prmt(vg, 0x64646464u, 0x4140u), 0x64806480u), sgi);
            r[4 * i + 1] = h2_mul(h2_sub(prmt(vg, 0x64646464u, 0x4342u), 0x64806480u), sgi);
            r[4 * i + 2] = h2_mul(h2_sub(prmt(vh, 0x64646464u, 0x4140u), 0x64806480u), shi);
            r[4 * i + 3] = h2_mul(h2_sub(prmt(vh, 0x64646464u, 0x4342u), 0x64806480u), shi);
        }
    } else {
        const uint4 sg4 = lds128(scr + g * 80 + 16 * P), sh4 = lds128(scr + (g + 8) * 80 + 16 * P);
        const uint32_t sg[4] = {sg4.x, sg4.y, sg4.z, sg4.w}, sh[4] = {sh4.x, sh4.y, sh4.z, sh4.w};
        uint4 u, hi = make_uint4(0, 0, 0, 0), hb = make_uint4(0, 0, 0, 0);
        if constexpr (FMT == KYB_FMT_Q6_K) {
            u = tr.q[P];
            hi = tr.q[4 + (P >> 1)];
        } else if constexpr (FMT == KYB_FMT_Q3_K) {
            u = tr.q[P >> 1];
            hb = tr.q[2];
        } else {
            u = tr.q[P];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int s = 4 * P + i;
            uint32_t g01, g23, h01, h23;                                                     // rows g / g + 8: weights (0, 1) and (2, 3) of the slice
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
                g01 = h2_sub(prmt(vg, 0x64646464u, 0x4140u), 0x64206420u), g23 = h2_sub(prmt(vg, 0x64646464u, 0x4342u), 0x64206420u);
                h01 = h2_sub(prmt(vh, 0x64646464u, 0x4140u), 0x64206420u), h23 = h2_sub(prmt(vh, 0x64646464u, 0x4342u), 0x64206420u);
            } else if constexpr (FMT == KYB_FMT_Q3_K) {
                uint32_t wg = (P & 1) ? u.z : u.x, wh = (P & 1) ? u.w : u.y;
                wg >>= 2 * i, wh >>= 2 * i;
                uint32_t bg = (P & 2) ? hb.z : hb.x, bh = (P & 2) ? hb.w : hb.y;
                const int i8 = s & 7;                                                        // bit i8 -> bit 2
                if (i8 < 2) bg <<= (2 - i8), bh <<= (2 - i8);
                else bg >>= (i8 - 2), bh >>= (i8 - 2);
                const uint32_t vg = and_or(wg, 0x03030303u, bg & 0x04040404u), vh = and_or(wh, 0x03030303u, bh & 0x04040404u);
                // (1024 + v) - 1028 = v - 4
                g01 = h2_sub(prmt(vg, 0x64646464u, 0x4140u), 0x64046404u), g23 = h2_sub(prmt(vg, 0x64646464u, 0x4342u), 0x64046404u);
                h01 = h2_sub(prmt(vh, 0x64646464u, 0x4140u), 0x64046404u), h23 = h2_sub(prmt(vh, 0x64646464u, 0x4342u), 0x64046404u);
            } else {
                const int p = i >> 1;
                const uint32_t wg = p ? u.z : u.x, wh = p ? u.w : u.y;
                uint32_t eg, og, eh, oh;                                                     // (w0, w2) and (w1, w3) as fp16 bits of value * 2^-14
                if ((i & 1) == 0) {
                    eg = wg & 0x8E008E00u, eh = wh & 0x8E008E00u;
                    og = (wg << 3) & 0x8E008E00u, oh = (wh << 3) & 0x8E008E00u;
                } else {
                    eg = and_or(wg << 6, 0x0E000E00u, (wg << 2) & 0x80008000u), eh = and_or(wh << 6, 0x0E000E00u, (wh << 2) & 0x80008000u);
                    og = and_or(wg << 9, 0x0E000E00u, (wg << 1) & 0x80008000u), oh = and_or(wh << 9, 0x0E000E00u, (wh << 1) & 0x80008000u);
                }
                eg = h2_mul(eg, 0x74007400u), og = h2_mul(og, 0x74007400u), eh = h2_mul(eh, 0x74007400u), oh = h2_mul(oh, 0x74007400u);   // * 2^14: the e2m1 value, exact
                g01 = prmt(eg, og, 0x5410u), g23 = prmt(eg, og, 0x7632u);
                h01 = prmt(eh, oh, 0x5410u), h23 = prmt(eh, oh, 0x7632u);
            }
            r[4 * i] = h2_mul(g01, sg[i]), r[4 * i + 1] = h2_mul(g23, sg[i]);
            r[4 * i + 2] = h2_mul(h01, sh[i]), r[4 * i + 3] = h2_mul(h23, sh[i]);
        }
    }
}

// The quarter's registers into the B stage. dst_g / dst_h: this lane's row addresses (8 (t & 1) already added). Under the 128-byte swizzle the 16-byte chunk of
// slice i sits at ((2 i + (t >> 1)) ^ g) * 16, and the 16 lanes an 8-byte store serves together have only four values of g: if all of them stored the same slice they
// would cover 4 distinct chunks (two-way bank conflict). So in step k the lanes with odd g store slice k ^ 2 instead of slice k: the 16 lanes then cover all 8
// chunks of their rows and every store is conflict-free. cxs[k] is the swizzled offset of the slice this lane stores in step k.
__device__ __forceinline__ void kq_store_quarter(uint32_t dst_g, uint32_t dst_h, const uint32_t (&cxs)[4], bool odd, const uint32_t (&r)[16]) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int a = 4 * k, b = 4 * (k ^ 2);
        sts64(dst_g + cxs[k], odd ? r[b] : r[a], odd ? r[b + 1] : r[a + 1]);
        sts64(dst_h + cxs[k], odd ? r[b + 2] : r[a + 2], odd ? r[b + 3] : r[a + 3]);
    }
}

// After quarter P of a tile has been computed, the registers it alone used are refilled from the next tile (in place: one register set, every unit is requested a
// whole tile ahead of its next use). Units shared by two quarters are refilled after the second one.
template <int FMT, int P>
__device__ __forceinline__ void kq_refill(const uint8_t* next, int lane, KqTile<FMT>& tr) {
    if constexpr (FMT == KYB_FMT_Q4_K || FMT == KYB_FMT_NVFP4 || FMT == KYB_FMT_IQ4_XS) {
        tr.q[P] = ldg128s(next + (P * 32 + lane) * 16);
    } else if constexpr (FMT == KYB_FMT_Q2_K) {
        if constexpr (P == 1) tr.q[0] = ldg128s(next + lane * 16);                           // 2-bit codes of quarters 0, 1
        if constexpr (P == 3) tr.q[1] = ldg128s(next + (32 + lane) * 16);
    } else if constexpr (FMT == KYB_FMT_Q5_K) {
        tr.q[P] = ldg128s(next + (P * 32 + lane) * 16);
        if constexpr (P == 1) {                                                              // fifth bits of quarters 0, 1
            const uint2 hb = ldg64s(next + 2048 + lane * 16);
            tr.q[4].x = hb.x, tr.q[4].y = hb.y;
        }
        if constexpr (P == 3) {
            const uint2 hb = ldg64s(next + 2048 + lane * 16 + 8);
            tr.q[4].z = hb.x, tr.q[4].w = hb.y;
        }
    } else if constexpr (FMT == KYB_FMT_Q8_0) {
        tr.q[2 * P] = ldg128s(next + (2 * P * 32 + lane) * 16);
        tr.q[2 * P + 1] = ldg128s(next + ((2 * P + 1) * 32 + lane) * 16);
    } else if constexpr (FMT == KYB_FMT_Q6_K) {
        tr.q[P] = ldg128s(next + (P * 32 + lane) * 16);
        if constexpr (P == 1) tr.q[4] = ldg128s(next + 2048 + lane * 16);                    // 2-bit planes of quarters 0, 1
        if constexpr (P == 3) tr.q[5] = ldg128s(next + 2048 + (32 + lane) * 16);             // ... of quarters 2, 3
    } else {
        if constexpr (P == 1) {
            tr.q[0] = ldg128s(next + lane * 16);                                             // 2-bit codes of quarters 0, 1 and their high bits
            const uint2 hb = ldg64s(next + 1024 + lane * 16);
            tr.q[2].x = hb.x, tr.q[2].y = hb.y;
        }
        if constexpr (P == 3) {
            tr.q[1] = ldg128s(next + (32 + lane) * 16);
            const uint2 hb = ldg64s(next + 1024 + lane * 16 + 8);
            tr.q[2].z = hb.x, tr.q[2].w = hb.y;
        }
    }
}

// The scale bytes of the next tile, requested once the scales of the current one have been prepared.
template <int FMT>
__device__ __forceinline__ void kq_refill_scales(const uint8_t* tile, int lane, KqTile<FMT>& tr) {
    const int r = lane >> 1, hf = lane & 1;
    if constexpr (FMT == KYB_FMT_Q4_K) {
        tr.sc = ldg128s(tile + 2048 + r * 16);
    } else if constexpr (FMT == KYB_FMT_Q5_K) {
        tr.sc = ldg128s(tile + 2560 + r * 16);
    } else if constexpr (FMT == KYB_FMT_Q8_0) {
        tr.sc = ldg128s(tile + 4096 + r * 16);
    } else if constexpr (FMT == KYB_FMT_Q2_K) {
        tr.sc = ldg128s(tile + 1024 + r * 16);
        tr.d16 = ldg32s(tile + 1280 + r * 4);
    } else if constexpr (FMT == KYB_FMT_IQ4_XS) {
        const uint2 mw = ldg64s(tile + 2048 + r * 8);
        tr.sc.x = mw.x, tr.sc.y = mw.y;
    } else if constexpr (FMT == KYB_FMT_Q6_K) {
        const uint2 s = ldg64s(tile + 3072 + r * 16 + 8 * hf);
        tr.sc.x = s.x, tr.sc.y = s.y;
        tr.d16 = ldg16s(tile + 3328 + r * 2);
    } else if constexpr (FMT == KYB_FMT_Q3_K) {
        const uint8_t* sp = tile + 1536 + r * 12;
        tr.sc.x = ldg32s(sp), tr.sc.y = ldg32s(sp + 4), tr.sc.z = ldg32s(sp + 8);
        tr.d16 = ldg16s(tile + 1728 + r * 2);
    } else {
        const uint2 s = ldg64s(tile + 2048 + r * 16 + 8 * hf);
        tr.sc.x = s.x, tr.sc.y = s.y;
    }
}

__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <int FMT>
__global__ void __launch_bounds__(KQ_THREADS, 1) gemm_kq_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ KqOutMaps outs, const KqParams p,
                                                                 const int num_items) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int TB = kyb_tile_bytes(FMT);
    const uint32_t a_bytes = (uint32_t)p.msub * KQ_A_SUB, stage_bytes = a_bytes + KQ_B_BYTES;
    const int STAGES = p.stages;
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t scr0 = smem0 + (uint32_t)STAGES * stage_bytes;
    const uint32_t stg0 = scr0 + KQ_DW * KQ_SCR;                                    // epilogue staging, 4 warps
    const uint32_t stg_bytes = p.wide ? 2 * KQ_STG : KQ_STG;
    const uint32_t bars = stg0 + 4 * stg_bytes;                                     // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], tmem slot
    const uint32_t full0 = bars, empty0 = bars + 8 * STAGES, accf0 = bars + 16 * STAGES, acce0 = accf0 + 16, tmem_slot = acce0 + 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t TMEM_COLS = 512;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init_a(full0 + 8 * s, KQ_DW + 1), mbar_init_a(empty0 + 8 * s, 1);
        for (int a = 0; a < 2; ++a) mbar_init_a(accf0 + 8 * a, 1), mbar_init_a(acce0 + 8 * a, 4);
        mbar_fence_init();
        prefetch_tmap(&tma_a);
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    // Grouped form with two-block items: a tile with more than 128 rows costs about 1.5 times a tile with fewer (eight MMAs per stage instead of four), and items go
    // to the CTAs round-robin, so the tiles are renumbered with the two-block ones first: every CTA then gets the same number of them (+-1) instead of a random
    // share. Warp 2 builds the table (two-block tiles from the front, the others from the back) from the segment offsets; more tiles than the table holds keep
    // their order.
    const uint16_t* tord = nullptr;
    if (p.tb && p.msub == 2) {
        const uint32_t total = p.tb[p.experts];
        if (total <= (uint32_t)KQ_TORD) {
            uint16_t* tw = reinterpret_cast<uint16_t*>(smem_raw + (tmem_slot + 16 - smem_u32(smem_raw)));
            tord = tw;
            if (warp == 2) {
                uint32_t front = 0, back = total;
                for (int e0 = 0; e0 < p.experts; e0 += 32) {
                    const int e = e0 + lane;
                    uint32_t two = 0, one = 0, first = 0;
                    if (e < p.experts) {
                        const uint32_t rows = p.off[e + 1] - p.off[e], nt = (rows + 255u) >> 8;
                        first = p.tb[e];
                        one = (nt && rows - 256u * (nt - 1u) <= 128u) ? 1u : 0u;
                        two = nt - one;
                    }
                    uint32_t a = two, b = one;                                          // inclusive warp scans
#pragma unroll
                    for (int d = 1; d < 32; d <<= 1) {
                        const uint32_t ua = __shfl_up_sync(0xffffffffu, a, d), ub = __shfl_up_sync(0xffffffffu, b, d);
                        if (lane >= d) a += ua, b += ub;
                    }
                    for (uint32_t i = 0; i < two; ++i) tw[front + a - two + i] = (uint16_t)(first + i);
                    if (one) tw[back - b] = (uint16_t)(first + two);
                    front += __shfl_sync(0xffffffffu, a, 31), back -= __shfl_sync(0xffffffffu, b, 31);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = lds32(tmem_slot);
    bool failed = false;

    if (warp == 0) {
        // ---- TMA producer: activation tiles
        if (elect_one()) {
            uint32_t parity = 1;                                                    // a fresh barrier passes a wait on the previous phase
            int s = 0;
            for (int t = blockIdx.x; t < num_items && !failed; t += gridDim.x) {
                const KqItem it = kq_item(p, t, tord);
                if (!it.valid) continue;
                for (int kb = 4 * it.tb0; kb < 4 * (it.tb0 + it.ntb) && !failed; ++kb) {
                    if (!mbar_wait_fast(empty0 + 8 * s, parity)) failed = true;
                    const uint32_t a_dst = smem0 + s * stage_bytes;
                    mbar_expect_tx_a(full0 + 8 * s, (uint32_t)it.nsub * KQ_A_SUB);
                    for (int sub = 0; sub < it.nsub; ++sub) tma_load_2d(a_dst + sub * KQ_A_SUB, &tma_a, kb * KQ_BK, it.m0 + sub * 128, full0 + 8 * s);
                    if (++s == STAGES) s = 0, parity ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (elect_one()) {
            constexpr uint32_t idesc = umma_idesc_f16(128, KQ_BN);
            uint32_t parity = 0;
            int s = 0;
            uint32_t cnt = 0;                                                       // accumulators used so far: number cnt lives in slot cnt & 1
            for (int t = blockIdx.x; t < num_items && !failed; t += gridDim.x) {
                const KqItem it = kq_item(p, t, tord);
                if (!it.valid) continue;
                // the epilogue must have drained an accumulator before the first MMA into it; the second block's accumulator is waited for only when its first MMA
                // is due, so the first stage of this item overlaps the tail of the previous item's epilogue
                if (!mbar_wait_fast(acce0 + 8 * (cnt & 1u), ((cnt >> 1) & 1u) ^ 1u)) failed = true;
                tc_fence_after();
                for (int kb = 0; kb < 4 * it.ntb && !failed; ++kb) {
                    if (!mbar_wait_fast(full0 + 8 * s, parity)) failed = true;
                    tc_fence_after();
                    const uint32_t a_src = smem0 + s * stage_bytes;
                    const uint64_t bdesc = umma_desc_sw128(a_src + a_bytes);
                    for (int sub = 0; sub < it.nsub; ++sub) {
                        const uint64_t adesc = umma_desc_sw128(a_src + sub * KQ_A_SUB);
                        const uint32_t tmem_d = tmem_base + (uint32_t)(((cnt + sub) & 1u) * KQ_BN);
                        if (kb == 0 && sub) {
                            if (!mbar_wait_fast(acce0 + 8 * ((cnt + 1u) & 1u), (((cnt + 1u) >> 1) & 1u) ^ 1u)) failed = true;
                            tc_fence_after();
                        }
#pragma unroll
                        for (int kk = 0; kk < KQ_BK / 16; ++kk) umma_f16(tmem_d, adesc + 2 * kk, bdesc + 2 * kk, idesc, (kb | kk) != 0);
                    }
                    umma_commit(empty0 + 8 * s);                                    // stage free once these MMAs have read it
                    if (++s == STAGES) s = 0, parity ^= 1u;
                }
                for (int sub = 0; sub < it.nsub; ++sub) umma_commit(accf0 + 8 * ((cnt + sub) & 1u));
                cnt += (uint32_t)it.nsub;
            }
        }
    } else if (warp < 6) {
        // ---- epilogue: warp w may touch TMEM lanes [32 (w % 4), 32 (w % 4) + 32)
        const int q = warp & 3;
        uint32_t cnt = 0;
        for (int t = blockIdx.x; t < num_items; t += gridDim.x) {
            const KqItem it = kq_item(p, t, tord);
            if (!it.valid) continue;
            for (int sub = 0; sub < it.nsub; ++sub, ++cnt) {
                const uint32_t slot = cnt & 1u;
                if (!mbar_wait_fast(accf0 + 8 * slot, (cnt >> 1) & 1u)) failed = true;
                tc_fence_after();
                const float gscale = it.gscale;
                if (p.part) {
                    // ---- split-k: this range's accumulator as it is (fp32) through the staged tiled stores; the tensor map covers part as 16-bit pairs, so a step of
                    // 32 rows x 16 fp32 columns is the same 32 x 64-byte box as a step of fp16 outputs. Rows past m land in the padding rows of the range.
                    const uint32_t stg = stg0 + (uint32_t)q * stg_bytes;
                    const int row0 = it.sp * p.mpad + it.m0 + sub * 128 + q * 32;
#pragma unroll 1
                    for (int c = 0; c < KQ_BN; c += 32) {
                        uint32_t v[32];
                        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + slot * KQ_BN + (uint32_t)c, v);
                        tmem_ld_wait();
                        uint32_t w[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) w[j] = v[j];
                        epilogue_stage_store(outs, 1, stg, lane, w, 2 * (it.n0 + c), row0, !failed);
#pragma unroll
                        for (int j = 0; j < 16; ++j) w[j] = v[16 + j];
                        epilogue_stage_store(outs, 1, stg, lane, w, 2 * (it.n0 + c + 16), row0, !failed);
                    }
                } else if (p.tma_out) {
                    // ---- staged tiled stores: 32 rows x 32 columns per step go to shared memory (64-byte swizzle, conflict-free 16-byte stores) and leave as one bulk
                    // tensor store per receiving rank: full 64-byte row segments on the wire, rows / columns past the matrix are dropped by the tensor map
                    const uint32_t stg = stg0 + (uint32_t)q * stg_bytes;
                    const int row0 = it.m0 + sub * 128 + q * 32;
#pragma unroll 1
                    for (int c = 0; c < KQ_BN; c += 32) {
                        uint32_t v[32];
                        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + slot * KQ_BN + (uint32_t)c, v);
                        tmem_ld_wait();
                        uint32_t w[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            __half2 h = sat_half2(__uint_as_float(v[2 * j]) * gscale, __uint_as_float(v[2 * j + 1]) * gscale);
                            w[j] = *reinterpret_cast<uint32_t*>(&h);
                        }
                        if (p.wide)
                            epilogue_stage_store_wide(outs, p.nout, stg, lane, w, (c >> 5) & 1, p.col0 + it.n0 + (c & ~63), row0,
                                                      !failed && row0 < it.m_end && it.n0 + (c & ~63) < p.n);
                        else
                            epilogue_stage_store(outs, p.nout, stg, lane, w, p.col0 + it.n0 + c, row0, !failed && row0 < it.m_end && it.n0 + c < p.n);
                    }
                } else if (p.tb && (p.ldd & 7) == 0 && ((uintptr_t)p.d[0] & 15) == 0) {
                    // ---- grouped form: rows end inside a tile or are scattered, so no tensor map fits. A step of 32 rows x 32 columns is transposed through the warp's
                    // staging buffer: every store instruction then writes 64-byte row segments (8 rows x 4 lanes) instead of 16 bytes of each of 32 rows
                    const uint32_t stg = stg0 + (uint32_t)q * stg_bytes;
                    const int row0 = it.m0 + sub * 128 + q * 32, row = row0 + lane;
                    const uint32_t orow = (p.row_map && row < it.m_end) ? p.row_map[row] : (uint32_t)row;
                    __half* dst[4];
                    bool live[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int rr = 8 * i + (lane >> 2);
                        const uint32_t o = __shfl_sync(0xffffffffu, orow, rr);
                        live[i] = row0 + rr < it.m_end && !failed;
                        dst[i] = p.d[0] + (size_t)o * p.ldd + it.n0 + 8 * (lane & 3);
                    }
#pragma unroll 1
                    for (int c = 0; c < (p.glu ? KQ_BN / 2 : KQ_BN); c += 32) {
                        uint32_t v[32], w[16];
                        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + slot * KQ_BN + (uint32_t)c, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            __half2 h = sat_half2(__uint_as_float(v[2 * i]) * gscale, __uint_as_float(v[2 * i + 1]) * gscale);
                            w[i] = *reinterpret_cast<uint32_t*>(&h);
                        }
                        if (p.glu) {
                            // w holds the gate products rounded to fp16 (what the reference's two-launch form would have stored); the up products of the same
                            // output columns sit 128 accumulator columns further
                            tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + slot * KQ_BN + (uint32_t)(KQ_BN / 2 + c), v);
                            tmem_ld_wait();
                            const float gsb = it.gscale_b, lim = p.limit;
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const __half2 a2 = *reinterpret_cast<__half2*>(&w[i]);
                                float a0 = __low2float(a2), a1 = __high2float(a2);
                                float b0 = __half2float(sat_half(__uint_as_float(v[2 * i]) * gsb)), b1 = __half2float(sat_half(__uint_as_float(v[2 * i + 1]) * gsb));
                                if (lim > 0.f) a0 = fminf(a0, lim), a1 = fminf(a1, lim), b0 = fminf(fmaxf(b0, -lim), lim), b1 = fminf(fmaxf(b1, -lim), lim);
                                __half2 h = sat_half2(a0 * (1.0f / (1.0f + expf(-a0))) * b0, a1 * (1.0f / (1.0f + expf(-a1))) * b1);
                                w[i] = *reinterpret_cast<uint32_t*>(&h);
                            }
                        }
                        __syncwarp();                                                  // the previous step's reads of the staging buffer are done
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            sts128(stg + (uint32_t)lane * 64u + (uint32_t)((j ^ ((lane >> 1) & 3)) << 4), make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]));
                        __syncwarp();
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int rr = 8 * i + (lane >> 2);
                            const uint4 o = lds128(stg + (uint32_t)rr * 64u + (uint32_t)(((lane & 3) ^ ((rr >> 1) & 3)) << 4));
                            if (live[i]) *reinterpret_cast<uint4*>(dst[i] + c) = o;
                        }
                    }
                } else {
                const int row = it.m0 + sub * 128 + q * 32 + lane;
                const size_t orow = (p.row_map && row < it.m_end) ? (size_t)p.row_map[row] : (size_t)row;
                const size_t doff = orow * p.ldd + it.n0;
#pragma unroll 1
                for (int c = 0; c < KQ_BN; c += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + slot * KQ_BN + (uint32_t)c, v);
                    tmem_ld_wait();
                    if (row < it.m_end && !failed) {
                        if (it.n0 + c + 32 <= p.n && (p.ldd & 7) == 0) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint4 o;
                                __half2 h0 = sat_half2(__uint_as_float(v[j]) * gscale, __uint_as_float(v[j + 1]) * gscale);
                                __half2 h1 = sat_half2(__uint_as_float(v[j + 2]) * gscale, __uint_as_float(v[j + 3]) * gscale);
                                __half2 h2 = sat_half2(__uint_as_float(v[j + 4]) * gscale, __uint_as_float(v[j + 5]) * gscale);
                                __half2 h3 = sat_half2(__uint_as_float(v[j + 6]) * gscale, __uint_as_float(v[j + 7]) * gscale);
                                o.x = *reinterpret_cast<uint32_t*>(&h0), o.y = *reinterpret_cast<uint32_t*>(&h1), o.z = *reinterpret_cast<uint32_t*>(&h2), o.w = *reinterpret_cast<uint32_t*>(&h3);
                                for (int pr = 0; pr < p.nout; ++pr) *reinterpret_cast<uint4*>(p.d[pr] + doff + c + j) = o;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (it.n0 + c + j < p.n)
                                    for (int pr = 0; pr < p.nout; ++pr) p.d[pr][doff + c + j] = sat_half(__uint_as_float(v[j]) * gscale);
                        }
                    }
                }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_a(acce0 + 8 * slot);                       // this warp has read its quarter of the accumulator
            }
        }
    } else {
        // ---- decoders
        const int dw = warp - 6, g = lane >> 2, tq = lane & 3;
        const uint32_t scr = scr0 + dw * KQ_SCR;
        // rows 16 dw + g and 16 dw + g + 8 of the B tile: 128-byte rows in 8-row groups of 1024 bytes, 16-byte chunks XOR-swizzled with the row number (row & 7 = g)
        const uint32_t row_off = (uint32_t)(2 * dw) * 1024u + (uint32_t)g * 128u + 8u * (uint32_t)(tq & 1);
        const bool odd = (g & 1) != 0;
        uint32_t cx[4];                                                              // offset of the slice this lane stores in step k (see kq_store_quarter)
#pragma unroll
        for (int i = 0; i < 4; ++i) cx[i] = (uint32_t)(((2 * (i ^ (odd ? 2 : 0)) + (tq >> 1)) ^ g) * 16);
        uint32_t parity = 1;
        int s = 0;
        for (int t = blockIdx.x; t < num_items && !failed; t += gridDim.x) {
            const KqItem it = kq_item(p, t, tord);
            if (!it.valid) continue;
            const int rt = min(it.b_rt0 + (p.glu ? (dw & 7) : dw), p.rt_total - 1);      // gated pair: warps 0-7 decode the gate rows, 8-15 the same rows of the up stack
            const uint8_t* tp = ((p.glu && dw >= 8) ? p.t16b : p.t16) + ((size_t)rt * (size_t)p.nb + (size_t)it.tb0) * TB;
            const int nbk = it.ntb;                                                      // 256-input blocks of this item
            // Software pipeline over the 64-input quarters: while the stores of quarter q drain into the stage (and before the proxy fence that publishes them), the
            // registers of quarter q + 1 are computed, so the wait for a free stage, the scale loads and the arithmetic overlap the shared-memory traffic.
            KqTile<FMT> tr;
            uint32_t r[16];
            kq_load<FMT>(tp, lane, tr);
            kq_prep_scales<FMT>(tr, scr, lane);
            __syncwarp();
            if (nbk > 1) kq_refill_scales<FMT>(tp + TB, lane, tr);
            kq_compute_quarter<FMT, 0>(tr, scr, lane, r);
            if (nbk > 1) kq_refill<FMT, 0>(tp + TB, lane, tr);
#define KYB_KQ_PUBLISH()                                                                                          \
    {                                                                                                             \
        fence_proxy_async_smem();                                                                                 \
        __syncwarp();                                                                                             \
        if (lane == 0) mbar_arrive_a(full0 + 8 * s);                                                              \
        if (++s == STAGES) s = 0, parity ^= 1u;                                                                   \
    }
#define KYB_KQ_STORE()                                                                                            \
    {                                                                                                             \
        if (!mbar_wait_fast(empty0 + 8 * s, parity)) failed = true;                                               \
        const uint32_t b_dst = smem0 + s * stage_bytes + a_bytes + row_off;                                       \
        kq_store_quarter(b_dst, b_dst + 1024u, cx, odd, r);                                                       \
    }
            for (int kb = 0; kb < nbk && !failed; ++kb) {
                const bool more = kb + 1 < nbk, more2 = kb + 2 < nbk;
                const uint8_t* nx = tp + (size_t)(kb + 1) * TB;                      // the next tile, two tiles ahead for the units already consumed
                KYB_KQ_STORE()
                kq_compute_quarter<FMT, 1>(tr, scr, lane, r);
                if (more) kq_refill<FMT, 1>(nx, lane, tr);
                KYB_KQ_PUBLISH()
                KYB_KQ_STORE()
                kq_compute_quarter<FMT, 2>(tr, scr, lane, r);
                if (more) kq_refill<FMT, 2>(nx, lane, tr);
                KYB_KQ_PUBLISH()
                KYB_KQ_STORE()
                kq_compute_quarter<FMT, 3>(tr, scr, lane, r);
                if (more) kq_refill<FMT, 3>(nx, lane, tr);
                KYB_KQ_PUBLISH()                                                     // its warp barrier also ends every lane's reads of this tile's scales
                if (more) {
                    kq_prep_scales<FMT>(tr, scr, lane);                              // tr.sc holds the next tile's scale bytes
                    __syncwarp();
                    if (more2) kq_refill_scales<FMT>(nx + TB, lane, tr);
                }
                KYB_KQ_STORE()
                if (more) {
                    kq_compute_quarter<FMT, 0>(tr, scr, lane, r);                    // quarter 0 of the next tile
                    if (more2) kq_refill<FMT, 0>(nx + TB, lane, tr);
                }
                KYB_KQ_PUBLISH()
            }
#undef KYB_KQ_PUBLISH
#undef KYB_KQ_STORE
        }
    }
    if (warp >= 2 && warp < 6 && lane == 0 && (p.tma_out || p.part)) tma_store_wait_all();   // the staging buffer must outlive its stores
    if (failed) atomicExch(p.status, KYB_DEV_TIMEOUT_GEMM);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}


// split-k, second step: d [m, n] = sat(gscale * (part[0] + part[1] + ... in k order)), eight columns per thread
__global__ void gemm_kq_reduce_kernel(const float* __restrict__ part, int ksplit, int m, int mpad, int n, int64_t ldp, float gscale, __half* __restrict__ d, int64_t ldd) {
    const int n8 = (n + 7) >> 3;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)m * n8) return;
    const int row = (int)(i / n8), c0 = (int)(i % n8) * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int sp = 0; sp < ksplit; ++sp) {
        const float4* src = reinterpret_cast<const float4*>(part + ((size_t)sp * (size_t)mpad + (size_t)row) * (size_t)ldp + c0);
        const float4 a = src[0], b = src[1];                                            // ldp is a multiple of 256: always inside the row
        acc[0] += a.x, acc[1] += a.y, acc[2] += a.z, acc[3] += a.w, acc[4] += b.x, acc[5] += b.y, acc[6] += b.z, acc[7] += b.w;
    }
    __half* dst = d + (size_t)row * (size_t)ldd + c0;
    if (c0 + 8 <= n && (ldd & 7) == 0 && ((uintptr_t)d & 15) == 0) {
        __half2 h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = sat_half2(acc[2 * j] * gscale, acc[2 * j + 1] * gscale);
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(h);
    } else {
        for (int j = 0; j < 8 && c0 + j < n; ++j) dst[j] = sat_half(acc[j] * gscale);
    }
}

// ------------------------------------------------------------------------------------------------ the dense form by CTA pairs (tcgen05 cta_group::2)
// A pair of CTAs computes a 256 x 256 tile of D: each CTA holds 128 activation rows (TMA) and decodes ONE HALF of the 256 weight rows (8 row tiles) of a
// 128-input stage; one MMA of the pair's leader runs on both tensor cores. Per SM and per flop the decode work, the decoder stores and the B operand reads are
// half of those of a one-CTA item with two activation blocks, which is what bounds that form (shared-memory bandwidth). The 16 decoder warps of a CTA are
// (row tile w & 7, quarter parity w >> 3): a warp decodes quarters hq and hq + 2 of every T16 tile of its row tile, one per stage (a stage is 128 inputs =
// two 64-input K-halves; quarter hq or hq + 2 of the tile lands in K-half hq). Barriers as in the NVFP4 pair kernel: full[s] in the leader (the leader's
// producer with the byte count of both CTAs' activation tiles + the 32 decoder warps of both CTAs, the peer's by remote arrive), empty[s] and acc_full in each
// CTA (commit to the pair), acc_empty in the leader (8 epilogue warps). Two accumulators alternate. Every wait is bounded.
// The decoder warps of the peer arrive on the leader's barrier with the plain (CTA-scope release) form of the remote arrive, as the vendor's own pipelines do
// for remote arrivals: by then the warp's stores sit in its own CTA's shared memory behind a proxy fence, which is where the leader's MMA reads them. With
// release at cluster scope on each of the 32 arrivals per stage the kernel ran at 950 TFLOP/s instead of 1430.
constexpr uint32_t KP_A_BYTES = 2 * KQ_A_SUB, KP_B_BYTES = 2 * 128 * KQ_BK * 2, KP_STAGE_BYTES = KP_A_BYTES + KP_B_BYTES;   // 32 K + 32 K per 128-input stage
constexpr int KP_STAGES = 3;

// registers that only quarter P of the tile used are refilled from the next tile right after P has been computed (this warp uses two quarters of a tile)
template <int FMT, int P>
__device__ __forceinline__ void kq_refill_pair(const uint8_t* next, int lane, KqTile<FMT>& tr) {
    if constexpr (FMT == KYB_FMT_Q4_K || FMT == KYB_FMT_NVFP4 || FMT == KYB_FMT_IQ4_XS) {
        tr.q[P] = ldg128s(next + (P * 32 + lane) * 16);
    } else if constexpr (FMT == KYB_FMT_Q2_K) {
        tr.q[P >> 1] = ldg128s(next + ((P >> 1) * 32 + lane) * 16);
    } else if constexpr (FMT == KYB_FMT_Q5_K) {
        tr.q[P] = ldg128s(next + (P * 32 + lane) * 16);
        const uint2 hb = ldg64s(next + 2048 + lane * 16 + ((P & 2) ? 8 : 0));
        if constexpr ((P & 2) == 0) tr.q[4].x = hb.x, tr.q[4].y = hb.y;
        else tr.q[4].z = hb.x, tr.q[4].w = hb.y;
    } else if constexpr (FMT == KYB_FMT_Q8_0) {
        tr.q[2 * P] = ldg128s(next + (2 * P * 32 + lane) * 16);
        tr.q[2 * P + 1] = ldg128s(next + ((2 * P + 1) * 32 + lane) * 16);
    } else if constexpr (FMT == KYB_FMT_Q6_K) {
        tr.q[P] = ldg128s(next + (P * 32 + lane) * 16);
        tr.q[4 + (P >> 1)] = ldg128s(next + 2048 + ((P >> 1) * 32 + lane) * 16);
    } else {
        tr.q[P >> 1] = ldg128s(next + ((P >> 1) * 32 + lane) * 16);
        const uint2 hb = ldg64s(next + 1024 + lane * 16 + ((P & 2) ? 8 : 0));
        if constexpr ((P & 2) == 0) tr.q[2].x = hb.x, tr.q[2].y = hb.y;
        else tr.q[2].z = hb.x, tr.q[2].w = hb.y;
    }
}

struct KpTile {
    int m0, n0;      // this CTA's first activation row, first weight row of the 256-wide tile
};
__device__ __forceinline__ KpTile kp_tile(const KqParams& p, int t, uint32_t rank) {
    KpTile it;
    const int tn = t / p.tiles_m, tm = t - tn * p.tiles_m;                          // m fastest: the pairs running together share the weight rows
    it.n0 = tn * KQ_BN, it.m0 = tm * 256 + (int)rank * 128;
    return it;
}

template <int FMT, int HQ>
__device__ __forceinline__ bool kp_decode(const KqParams& p, const int num_items, const int pair, const int pairs, const uint32_t rank, const int rt8, const int lane,
                                          const uint32_t smem0, const uint32_t scr, const uint32_t full_leader0, const uint32_t empty0) {
    constexpr int TB = kyb_tile_bytes(FMT);
    const int g = lane >> 2, tq = lane & 3;
    const uint32_t row_off = (uint32_t)(2 * rt8) * 1024u + (uint32_t)g * 128u + 8u * (uint32_t)(tq & 1);
    const bool odd = (g & 1) != 0;
    uint32_t cx[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) cx[i] = (uint32_t)(((2 * (i ^ (odd ? 2 : 0)) + (tq >> 1)) ^ g) * 16);
    uint32_t parity = 1;
    int s = 0;
    bool failed = false;
    for (int t = pair; t < num_items && !failed; t += pairs) {
        const KpTile it = kp_tile(p, t, rank);
        const int rt = min((it.n0 >> 4) + (int)rank * 8 + rt8, p.rt_total - 1);
        const uint8_t* tp = p.t16 + (size_t)rt * (size_t)p.nb * TB;
        KqTile<FMT> tr;
        uint32_t r[16];
        kq_load<FMT>(tp, lane, tr);
        kq_prep_scales<FMT>(tr, scr, lane);
        __syncwarp();
        if (p.nb > 1) kq_refill_scales<FMT>(tp + TB, lane, tr);
        kq_compute_quarter<FMT, HQ>(tr, scr, lane, r);
        if (p.nb > 1) kq_refill_pair<FMT, HQ>(tp + TB, lane, tr);
#define KYB_KP_STORE()                                                                                            \
    {                                                                                                             \
        if (!mbar_wait_fast(empty0 + 8 * s, parity)) failed = true;                                               \
        const uint32_t b_dst = smem0 + s * KP_STAGE_BYTES + KP_A_BYTES + HQ * 16384u + row_off;                   \
        kq_store_quarter(b_dst, b_dst + 1024u, cx, odd, r);                                                       \
    }
#define KYB_KP_PUBLISH()                                                                                          \
    {                                                                                                             \
        fence_proxy_async_smem();                                                                                 \
        __syncwarp();                                                                                             \
        if (lane == 0) mbar_arrive_remote(full_leader0 + 8 * s);                                                  \
        if (++s == KP_STAGES) s = 0, parity ^= 1u;                                                                \
    }
        for (int kb = 0; kb < p.nb && !failed; ++kb) {
            const bool more = kb + 1 < p.nb, more2 = kb + 2 < p.nb;
            const uint8_t* nx = tp + (size_t)(kb + 1) * TB;
            KYB_KP_STORE()                                                       // quarter HQ: inputs [0, 128) of the tile
            kq_compute_quarter<FMT, HQ + 2>(tr, scr, lane, r);
            if (more) kq_refill_pair<FMT, HQ + 2>(nx, lane, tr);
            KYB_KP_PUBLISH()                                                     // its warp barrier also ends every lane's reads of this tile's scales
            if (more) {
                kq_prep_scales<FMT>(tr, scr, lane);                              // tr.sc holds the next tile's scale bytes
                __syncwarp();
                if (more2) kq_refill_scales<FMT>(nx + TB, lane, tr);
            }
            KYB_KP_STORE()                                                       // quarter HQ + 2: inputs [128, 256)
            if (more) {
                kq_compute_quarter<FMT, HQ>(tr, scr, lane, r);
                if (more2) kq_refill_pair<FMT, HQ>(nx + TB, lane, tr);
            }
            KYB_KP_PUBLISH()
        }
#undef KYB_KP_STORE
#undef KYB_KP_PUBLISH
    }
    return failed;
}

template <int FMT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(KQ_THREADS, 1)
    gemm_kq_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ KqOutMaps outs, const KqParams p, const int num_items) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t scr0 = smem0 + (uint32_t)KP_STAGES * KP_STAGE_BYTES;
    const uint32_t stg0 = scr0 + KQ_DW * KQ_SCR;                                    // epilogue staging, 4 warps
    const uint32_t bars = stg0 + 4 * KQ_STG;                                        // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], tmem slot
    const uint32_t full0 = bars, empty0 = bars + 8 * KP_STAGES, accf0 = bars + 16 * KP_STAGES, acce0 = accf0 + 16, tmem_slot = acce0 + 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair = (int)(blockIdx.x >> 1), pairs = (int)(gridDim.x >> 1);
    const int kstages = p.k / 128;
    constexpr uint32_t TMEM_COLS = 512;

    if (threadIdx.x == 0) {
        for (int s = 0; s < KP_STAGES; ++s) mbar_init_a(full0 + 8 * s, 2 * KQ_DW + 1), mbar_init_a(empty0 + 8 * s, 1);
        for (int a = 0; a < 2; ++a) mbar_init_a(accf0 + 8 * a, 1), mbar_init_a(acce0 + 8 * a, 8);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&tma_a);
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tc_fence_before();
    cluster_sync_all();                                                            // both CTAs' barriers exist before either signals the other
    tc_fence_after();
    const uint32_t tmem_base = lds32(tmem_slot);
    const uint32_t full_leader0 = map_to_rank(full0, 0);
    bool failed = false;

    if (warp == 0) {
        // ---- TMA producer: this CTA's 128 activation rows, two 64-input boxes per stage
        if (elect_one()) {
            uint32_t parity = 1;
            int s = 0;
            for (int t = pair; t < num_items && !failed; t += pairs) {
                const KpTile it = kp_tile(p, t, rank);
                for (int ks = 0; ks < kstages && !failed; ++ks) {
                    if (!mbar_wait_fast(empty0 + 8 * s, parity)) failed = true;
                    const uint32_t a_dst = smem0 + s * KP_STAGE_BYTES;
                    if (rank == 0) mbar_expect_tx_a(full0 + 8 * s, 2 * KP_A_BYTES);
                    tma_load_2d_pair(a_dst, &tma_a, ks * 128, it.m0, full_leader0 + 8 * s);
                    tma_load_2d_pair(a_dst + KQ_A_SUB, &tma_a, ks * 128 + 64, it.m0, full_leader0 + 8 * s);
                    if (++s == KP_STAGES) s = 0, parity ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: the pair's leader
        if (rank == 0 && elect_one()) {
            constexpr uint32_t idesc = umma_idesc_f16(256, KQ_BN);
            uint32_t parity = 0;
            int s = 0;
            uint32_t cnt = 0;
            for (int t = pair; t < num_items && !failed; t += pairs, ++cnt) {
                const uint32_t slot = cnt & 1u;
                if (!mbar_wait_fast(acce0 + 8 * slot, ((cnt >> 1) & 1u) ^ 1u)) failed = true;           // both CTAs' epilogues have drained the slot
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + slot * KQ_BN;
                for (int ks = 0; ks < kstages && !failed; ++ks) {
                    if (!mbar_wait_fast(full0 + 8 * s, parity)) failed = true;
                    tc_fence_after();
                    const uint32_t a_src = smem0 + s * KP_STAGE_BYTES, b_src = a_src + KP_A_BYTES;
#pragma unroll
                    for (int kh = 0; kh < 2; ++kh) {
                        const uint64_t adesc = umma_desc_sw128(a_src + kh * KQ_A_SUB), bdesc = umma_desc_sw128(b_src + kh * 16384u);
#pragma unroll
                        for (int kk = 0; kk < KQ_BK / 16; ++kk) umma_f16_pair(tmem_d, adesc + 2 * kk, bdesc + 2 * kk, idesc, (ks | kh | kk) != 0);
                    }
                    umma_commit_pair(empty0 + 8 * s);
                    if (++s == KP_STAGES) s = 0, parity ^= 1u;
                }
                umma_commit_pair(accf0 + 8 * slot);
            }
        }
    } else if (warp < 6) {
        // ---- epilogue: this CTA's 128 rows x 256 columns, staged tiled bulk stores
        const int q = warp & 3;
        const uint32_t acce_leader0 = map_to_rank(acce0, 0);
        uint32_t cnt = 0;
        for (int t = pair; t < num_items; t += pairs, ++cnt) {
            const KpTile it = kp_tile(p, t, rank);
            const uint32_t slot = cnt & 1u;
            if (!mbar_wait_fast(accf0 + 8 * slot, (cnt >> 1) & 1u)) failed = true;
            tc_fence_after();
            const uint32_t stg = stg0 + (uint32_t)q * KQ_STG;
            const int row0 = it.m0 + q * 32;
#pragma unroll 1
            for (int c = 0; c < KQ_BN; c += 32) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + slot * KQ_BN + (uint32_t)c, v);
                tmem_ld_wait();
                uint32_t w[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    __half2 h = sat_half2(__uint_as_float(v[2 * j]) * p.gscale, __uint_as_float(v[2 * j + 1]) * p.gscale);
                    w[j] = *reinterpret_cast<uint32_t*>(&h);
                }
                epilogue_stage_store(outs, 1, stg, lane, w, it.n0 + c, row0, !failed && row0 < p.m && it.n0 + c < p.n);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acce_leader0 + 8 * slot);
        }
    } else {
        // ---- decoders
        const int dw = warp - 6;
        const uint32_t scr = scr0 + dw * KQ_SCR;
        if (dw < 8) failed = kp_decode<FMT, 0>(p, num_items, pair, pairs, rank, dw, lane, smem0, scr, full_leader0, empty0);
        else failed = kp_decode<FMT, 1>(p, num_items, pair, pairs, rank, dw - 8, lane, smem0, scr, full_leader0, empty0);
    }
    if (warp >= 2 && warp < 6 && lane == 0) tma_store_wait_all();                      // the staging buffer must outlive its stores
    if (failed) atomicExch(p.status, KYB_DEV_TIMEOUT_GEMM);
    tc_fence_before();
    cluster_sync_all();                                                            // neither CTA frees tensor memory or leaves while the other may still signal it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

}  // namespace kyb

namespace {

int kq_launch(int fmt, const CUtensorMap& ta, const KybOutMaps& outs, kyb::KqParams p, int num_items, cudaStream_t st) {
    static std::mutex mu;
    static unsigned done[KYB_FMT_COUNT] = {};
    static int sms = 0;
    int dev = 0;
    KYB_CUDA(cudaGetDevice(&dev));
    const void* kern = fmt == KYB_FMT_Q4_K   ? (const void*)kyb::gemm_kq_kernel<KYB_FMT_Q4_K>
                       : fmt == KYB_FMT_Q6_K ? (const void*)kyb::gemm_kq_kernel<KYB_FMT_Q6_K>
                       : fmt == KYB_FMT_Q3_K ? (const void*)kyb::gemm_kq_kernel<KYB_FMT_Q3_K>
                       : fmt == KYB_FMT_Q5_K ? (const void*)kyb::gemm_kq_kernel<KYB_FMT_Q5_K>
                       : fmt == KYB_FMT_Q8_0 ? (const void*)kyb::gemm_kq_kernel<KYB_FMT_Q8_0>
                       : fmt == KYB_FMT_Q2_K ? (const void*)kyb::gemm_kq_kernel<KYB_FMT_Q2_K>
                       : fmt == KYB_FMT_IQ4_XS ? (const void*)kyb::gemm_kq_kernel<KYB_FMT_IQ4_XS>
                                             : (const void*)kyb::gemm_kq_kernel<KYB_FMT_NVFP4>;
    const uint32_t stage_bytes = (uint32_t)p.msub * kyb::KQ_A_SUB + kyb::KQ_B_BYTES;
    const size_t fixed = (size_t)kyb::KQ_DW * kyb::KQ_SCR + 4 * (p.wide ? 2 : 1) * kyb::KQ_STG + 1024 + 256 + (p.tb ? 2 * kyb::KQ_TORD : 0);
    const size_t cap = 227 * 1024;
    p.stages = (int)std::min<size_t>(8, (cap - fixed) / stage_bytes);
    const size_t smem = (size_t)p.stages * stage_bytes + fixed;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!(done[fmt] & (1u << (dev & 31)))) {
            KYB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cap));
            done[fmt] |= 1u << (dev & 31);
        }
        if (!sms) KYB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    }
    void* args[] = {(void*)&ta, (void*)&outs, (void*)&p, (void*)&num_items};
    KYB_CUDA(cudaLaunchKernel(kern, dim3((unsigned)std::min(num_items, sms)), dim3(kyb::KQ_THREADS), args, smem, st));
    return kyb_launch_check("gemm_kq");
}

// the dense form by CTA pairs; KYB_EUNSUPPORTED when the device cannot hold a pair of these CTAs at once or the tile count suits the one-CTA kernel better (the
// caller then takes that kernel)
int kq_launch_pair(int fmt, const CUtensorMap& ta, const KybOutMaps& outs, kyb::KqParams p, cudaStream_t st) {
    static std::mutex mu;
    static unsigned done[KYB_FMT_COUNT] = {};
    static int pairs_max[KYB_FMT_COUNT][32] = {};
    int dev = 0;
    KYB_CUDA(cudaGetDevice(&dev));
    const void* kern = fmt == KYB_FMT_Q4_K   ? (const void*)kyb::gemm_kq_pair_kernel<KYB_FMT_Q4_K>
                       : fmt == KYB_FMT_Q6_K ? (const void*)kyb::gemm_kq_pair_kernel<KYB_FMT_Q6_K>
                       : fmt == KYB_FMT_Q3_K ? (const void*)kyb::gemm_kq_pair_kernel<KYB_FMT_Q3_K>
                       : fmt == KYB_FMT_Q5_K ? (const void*)kyb::gemm_kq_pair_kernel<KYB_FMT_Q5_K>
                       : fmt == KYB_FMT_Q8_0 ? (const void*)kyb::gemm_kq_pair_kernel<KYB_FMT_Q8_0>
                       : fmt == KYB_FMT_Q2_K ? (const void*)kyb::gemm_kq_pair_kernel<KYB_FMT_Q2_K>
                       : fmt == KYB_FMT_IQ4_XS ? (const void*)kyb::gemm_kq_pair_kernel<KYB_FMT_IQ4_XS>
                                             : (const void*)kyb::gemm_kq_pair_kernel<KYB_FMT_NVFP4>;
    constexpr size_t smem = (size_t)kyb::KP_STAGES * kyb::KP_STAGE_BYTES + (size_t)kyb::KQ_DW * kyb::KQ_SCR + 4 * kyb::KQ_STG + 1024 + 256;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!(done[fmt] & (1u << (dev & 31)))) {
            KYB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            cudaLaunchConfig_t qc = {};
            qc.gridDim = dim3(2), qc.blockDim = dim3(kyb::KQ_THREADS), qc.dynamicSmemBytes = smem;
            int nc = 0;
            if (cudaOccupancyMaxActiveClusters(&nc, kern, &qc) != cudaSuccess || nc <= 0) {
                (void)cudaGetLastError();
                nc = 0;
            }
            pairs_max[fmt][dev & 31] = nc;
            done[fmt] |= 1u << (dev & 31);
        }
    }
    const int pm = pairs_max[fmt][dev & 31];
    if (pm <= 0) return KYB_EUNSUPPORTED;
    p.msub = 2;
    p.tiles_m = (p.m + 255) / 256;
    const int num_items = p.tiles_n * p.tiles_m;
    // more tiles than pairs but no more than SMs: the one-CTA kernel runs them all at once, pairs would need a second, poorly filled wave (12288 -> 3072 at
    // M = 2048: 96 tiles, 156 us against 170 us)
    if (num_items > pm && num_items <= 2 * pm) return KYB_EUNSUPPORTED;
    const int pairs = std::min(num_items, pm);
    void* args[] = {(void*)&ta, (void*)&outs, (void*)&p, (void*)&num_items};
    KYB_CUDA(cudaLaunchKernel(kern, dim3((unsigned)(2 * pairs)), dim3(kyb::KQ_THREADS), args, smem, st));
    return kyb_launch_check("gemm_kq_pair");
}

}  // namespace

static int kq_dense(int fmt, const void* t16, int64_t n, int64_t k, const void* a, int64_t lda, int64_t m, float gscale, void* const* d, int nout, int64_t ldd,
                    int64_t col0, int msub, void* stream, bool pair_ok = true, int ksplit = 1, float* part = nullptr) {
    KYB_REQUIRE(fmt >= 0 && fmt < KYB_FMT_COUNT, "unknown weight format %d", fmt);
    KYB_REQUIRE(t16 && a, "null pointer");
    KYB_REQUIRE(m > 0 && n > 0 && k > 0 && k % 256 == 0, "m=%lld n=%lld k=%lld: k must be a positive multiple of 256", (long long)m, (long long)n, (long long)k);
    KYB_REQUIRE(lda >= k && lda % 8 == 0 && ldd >= n, "leading dimensions: lda >= k and a multiple of 8, ldd >= n");
    KYB_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)t16 & 15) == 0, "a and t16 must be 16-byte aligned");
    KYB_REQUIRE(m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 24), "dimension too large");
    KYB_REQUIRE(msub >= 0 && msub <= 2, "msub is 0 (automatic), 1 or 2");
    const bool automatic = msub == 0;                                              // a given msub asks for the one-CTA kernel with that many activation blocks per item
    unsigned int* status = kyb_device_status_word();
    KYB_REQUIRE(status, "could not set up the device status word");
    CUtensorMap ta;
    if (int rc = kyb_make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a, (uint64_t)m, (uint64_t)k, (uint64_t)lda * 2, 128, kyb::KQ_BK)) return rc;
    kyb::KqParams p;
    p.t16 = (const uint8_t*)t16, p.ldd = ldd, p.m = (int)m, p.n = (int)n, p.k = (int)k, p.nb = (int)(k / 256), p.rt_total = (int)((n + 15) / 16);
    p.nout = nout;
    for (int i = 0; i < 8; ++i) p.d[i] = i < nout ? (__half*)d[i] + col0 : nullptr;
    p.gscale = gscale, p.status = status, p.tb = nullptr, p.off = nullptr, p.row_map = nullptr, p.gs = nullptr, p.experts = 0;
    p.tiles_n = (int)((n + kyb::KQ_BN - 1) / kyb::KQ_BN);
    p.ksplit = ksplit, p.mpad = 0, p.part = ksplit > 1 ? part : nullptr, p.ldp = (int64_t)p.tiles_n * kyb::KQ_BN;
    if (!msub) {
        // two activation blocks per item halve the decode work per flop, but they halve the number of items and keep both accumulators busy (no overlap of
        // the epilogue with the next item): one block when the rows fit one block, when two-block items would leave more than half of the SMs idle, or when the
        // epilogue also feeds other GPUs (its peer stores then overlap the next item's MMAs)
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) (void)cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const int64_t items2 = (int64_t)p.tiles_n * ((m + 255) / 256);
        msub = (m <= 128 || items2 * 2 < sms || nout > 1) ? 1 : 2;
    }
    p.msub = msub;
    p.tiles_m = (int)((m + 128 * p.msub - 1) / (128 * p.msub));
    // tiled bulk stores need 16-byte aligned bases and row pitches; otherwise the epilogue stores from registers
    KybOutMaps outs;
    memset(&outs, 0, sizeof(outs));
    p.col0 = (int)col0;
    p.tma_out = (ldd % 8 == 0 && col0 % 8 == 0) ? 1 : 0;
    for (int i = 0; i < nout && p.tma_out; ++i)
        if ((uintptr_t)d[i] & 15) p.tma_out = 0;
    p.wide = (p.tma_out && nout > 1) ? 1 : 0;
    p.t16b = nullptr, p.gsb = nullptr, p.glu = 0, p.limit = 0.f;
    for (int i = 0; i < nout && p.tma_out; ++i)
        if (int rc = kyb_make_tmap_2d(&outs.m[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, d[i], (uint64_t)m, (uint64_t)(col0 + n), (uint64_t)ldd * 2, 32, p.wide ? 64 : 32,
                                      p.wide ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B))
            return rc;
    if (ksplit > 1) {
        // split-k: the one-CTA kernel over (tile, k-range) items, whose staged stores go to the fp32 ranges (tensor map over part as 16-bit pairs), then the
        // ranges are added
        p.mpad = p.tiles_m * 128 * p.msub, p.tma_out = 0, p.wide = 0;
        memset(&outs, 0, sizeof(outs));
        if (int rc = kyb_make_tmap_2d(&outs.m[0], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, part, (uint64_t)ksplit * (uint64_t)p.mpad, (uint64_t)(2 * p.ldp), (uint64_t)p.ldp * 4, 32, 32,
                                      CU_TENSOR_MAP_SWIZZLE_64B))
            return rc;
        if (int rc = kq_launch(fmt, ta, outs, p, p.tiles_n * p.tiles_m * ksplit, (cudaStream_t)stream)) return rc;
        const int64_t threads = m * ((n + 7) / 8);
        kyb::gemm_kq_reduce_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(part, ksplit, (int)m, p.mpad, (int)n, p.ldp, gscale, (__half*)d[0], ldd);
        return kyb_launch_check("gemm_kq_reduce");
    }
    if (nout == 1 && p.tma_out && m > 128 && pair_ok && automatic) {
        // one destination and at least two row blocks: CTA pairs (cta_group::2), each CTA decoding half of the 256 weight rows of a tile
        if (int rc = kq_launch_pair(fmt, ta, outs, p, (cudaStream_t)stream); rc != KYB_EUNSUPPORTED) return rc;
    }
    return kq_launch(fmt, ta, outs, p, p.tiles_n * p.tiles_m, (cudaStream_t)stream);
}

// D fp16 [m, n] (row stride ldd) = sat(gscale * A fp16 [m, k] (row stride lda) x W^T), W = T16 tiles of an [n, k] matrix of format fmt. msub = 0: the library
// chooses (CTA pairs for more than 128 rows, else the one-CTA kernel); 1 or 2: the one-CTA kernel with that many blocks of 128 activation rows per work item.
// All forms give the same bits.
extern "C" int kyb_gemm_kq(int fmt, const void* t16, int64_t n, int64_t k, const void* a, int64_t lda, int64_t m, float gscale, void* d, int64_t ldd, int msub,
                           void* stream) {
    KYB_REQUIRE(d && ((uintptr_t)d & 1) == 0, "null or odd output pointer");
    void* outs[1] = {d};
    return kq_dense(fmt, t16, n, k, a, lda, m, gscale, outs, 1, ldd, 0, msub, stream);
}

// Split-k for products with fewer output tiles than SMs (e.g. 2048 x 3072 outputs from 12288 inputs: 96 tiles of 256 x 256): the k-blocks are cut into `split`
// equal ranges, (tile, range) items fill the SMs, every item leaves its fp32 accumulator in the workspace and a second kernel adds the ranges in k order (the result
// is deterministic; it differs from the unsplit product by fp32 summation order only). kyb_gemm_kq_split: the factor the library suggests (1: do not split);
// kyb_gemm_kq_split_bytes: bytes of 16-byte aligned workspace the call then needs.
extern "C" int kyb_gemm_kq_split(int fmt, int64_t n, int64_t k, int64_t m) {
    if (fmt < 0 || fmt >= KYB_FMT_COUNT || n <= 0 || k <= 0 || k % 256 || m <= 128) return 1;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) (void)cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    (void)cudaGetLastError();
    const int64_t tiles = ((n + 255) / 256) * ((m + 255) / 256), nb = k / 256;
    if (tiles >= sms) return 1;                                                       // whole rounds of tiles already fill the SMs
    // Cost model in microseconds, fitted to measurements with 2048 rows on 3072 x 12288, 1536 x 12288 and 768 x 12288: a 64-input stage of a two-block item of
    // the one-CTA kernel takes 0.73 us, a 128-input stage of the pair kernel 0.87 us, an item 6 us more (start, exposed epilogue); the split form pays about 10 us
    // for its second launch and moves (ranges + 0.5) x the fp32 output at about 3 MB per us. The unsplit product is whichever kernel the launcher would take
    // (pairs unless the tile count lies between the pair count and the SM count). A split must be at least 15 % faster than that.
    const double out_mb = (double)(((m + 255) / 256) * 256) * (double)(((n + 255) / 256) * 256) * 4.0 / 1.0e6;
    const int64_t pairs = sms / 2;
    double whole = 4.0 * nb * 0.73 + 6.0;                                              // fewer tiles than SMs: one round
    if (!(tiles > pairs && tiles <= 2 * pairs)) whole = std::min(whole, (double)((tiles + pairs - 1) / pairs) * (2.0 * nb * 0.87 + 6.0));
    int best = 1;
    double best_cost = 0.85 * whole;
    for (int sp = 2; sp <= 8; ++sp) {
        if (nb % sp || nb / sp < 8) continue;                                           // equal ranges of at least 2048 inputs
        const double rounds = (double)((tiles * sp + sms - 1) / sms);
        const double cost = rounds * (4.0 * (double)(nb / sp) * 0.73 + 6.0) + 10.0 + (sp + 0.5) * out_mb / 3.0;
        if (cost < best_cost) best = sp, best_cost = cost;
    }
    return best;
}
extern "C" size_t kyb_gemm_kq_split_bytes(int64_t n, int64_t m, int split) {
    if (n <= 0 || m <= 0 || split <= 1) return 0;
    return (size_t)split * (size_t)(((m + 255) / 256) * 256) * (size_t)(((n + 255) / 256) * 256) * sizeof(float);   // rows and columns padded to whole work items
}
extern "C" int kyb_gemm_kq_splitk(int fmt, const void* t16, int64_t n, int64_t k, const void* a, int64_t lda, int64_t m, float gscale, void* d, int64_t ldd, int split,
                                  void* workspace, size_t workspace_bytes, void* stream) {
    KYB_REQUIRE(d && ((uintptr_t)d & 1) == 0, "null or odd output pointer");
    KYB_REQUIRE(split >= 2 && split <= 8 && k > 0 && k % 256 == 0 && (k / 256) % split == 0, "split=%d: 2..8 equal ranges of whole 256-input blocks (k=%lld)", split, (long long)k);
    const size_t need = kyb_gemm_kq_split_bytes(n, m, split);
    if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 15)) {
        kyb_set_error("split-k needs %zu bytes of 16-byte aligned workspace, got %zu", need, workspace ? workspace_bytes : (size_t)0);
        return KYB_EWORKSPACE;
    }
    void* outs[1] = {d};
    return kq_dense(fmt, t16, n, k, a, lda, m, gscale, outs, 1, ldd, 0, m > 128 ? 2 : 1, stream, false, split, (float*)workspace);
}

// The same product with the all-gather of an N-sharded linear folded into the epilogue: every tile goes to the output matrix of every rank, at column col0.
extern "C" int kyb_gemm_kq_ag(int fmt, const void* t16, int64_t n, int64_t k, const void* a, int64_t lda, int64_t m, float gscale, const kyb_peer_out* out, int64_t ldd,
                              int64_t col0, int msub, void* stream) {
    KYB_REQUIRE(out && out->count >= 1 && out->count <= 8, "peer outputs: 1..8 ranks");
    KYB_REQUIRE(col0 >= 0 && col0 % 8 == 0 && col0 + n <= ldd && ldd % 8 == 0, "col0=%lld: a multiple of 8 with col0 + n <= ldd, ldd a multiple of 8", (long long)col0);
    void* outs[8];
    for (int i = 0; i < out->count; ++i) {
        KYB_REQUIRE(out->ptr[i] && ((uintptr_t)out->ptr[i] & 15) == 0, "peer output %d is null or not 16-byte aligned", i);
        outs[i] = out->ptr[i];
    }
    return kq_dense(fmt, t16, n, k, a, lda, m, gscale, outs, out->count, ldd, col0, msub, stream);
}

// Grouped form for routed experts: a fp16 [s, k] rows sorted by expert (segment e = rows [off[e], off[e + 1])), T16 of the expert stack (experts * n rows),
// tb / off from kyb_moe_plan with the same mt (128 or 256 rows of one expert per work item: with 256 a decoded weight tile serves up to two 128-row blocks, so an
// expert with 129..256 rows is decoded once, not twice), row_map (optional, u32 [s]) = output row of each sorted row, gs (optional) per-expert output scale.
// d [*, n]. The item list is sized for the worst case (s / mt + experts tiles per 256 output columns); items past tb[experts] are skipped.
// t16b != null: the gated pair. t16 / t16b are the gate and up stacks of one shape, d [s, n] = fp16(silu(a) * b) of their fp16-rounded products.
static int kq_grouped(int fmt, const void* t16, const void* t16b, int64_t n, int64_t k, int experts, const void* a, int64_t lda, int64_t s, const void* tb, const void* off,
                      const void* row_map, const void* gs, const void* gsb, float limit, void* d, int64_t ldd, int mt, void* stream) {
    const bool glu = t16b != nullptr;
    KYB_REQUIRE(mt == 128 || mt == 256, "mt=%d: 128 or 256 rows per work item", mt);
    KYB_REQUIRE(fmt >= 0 && fmt < KYB_FMT_COUNT, "unknown weight format %d", fmt);
    KYB_REQUIRE(t16 && a && d && tb && off, "null pointer");
    KYB_REQUIRE(s > 0 && n > 0 && k > 0 && k % 256 == 0 && experts > 0, "s=%lld n=%lld k=%lld experts=%d: k must be a positive multiple of 256", (long long)s, (long long)n,
                (long long)k, experts);
    if (glu) {
        KYB_REQUIRE(n % 128 == 0, "the gated pair needs n %% 128 == 0, got n=%lld", (long long)n);
        KYB_REQUIRE(ldd % 8 == 0 && ((uintptr_t)d & 15) == 0 && ((uintptr_t)t16b & 15) == 0 && !row_map, "the gated pair stores 16-byte pieces in sorted order: ldd %% 8 == 0, aligned d, no row_map");
    } else {
        KYB_REQUIRE(n % 256 == 0, "the grouped product needs n %% 256 == 0 (an output tile must not straddle two experts), got n=%lld", (long long)n);
    }
    KYB_REQUIRE(lda >= k && lda % 8 == 0 && ldd >= n, "leading dimensions: lda >= k and a multiple of 8, ldd >= n");
    KYB_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)t16 & 15) == 0, "a and t16 must be 16-byte aligned");
    KYB_REQUIRE(s < (1ll << 31) && (int64_t)experts * n < (1ll << 31) && k < (1ll << 24), "dimension too large");
    unsigned int* status = kyb_device_status_word();
    KYB_REQUIRE(status, "could not set up the device status word");
    CUtensorMap ta;
    if (int rc = kyb_make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a, (uint64_t)s, (uint64_t)k, (uint64_t)lda * 2, 128, kyb::KQ_BK)) return rc;
    kyb::KqParams p;
    p.t16 = (const uint8_t*)t16, p.ldd = ldd, p.m = (int)s, p.n = (int)n, p.k = (int)k, p.nb = (int)(k / 256);
    p.nout = 1;
    for (int i = 0; i < 8; ++i) p.d[i] = i == 0 ? (__half*)d : nullptr;
    p.rt_total = (int)((int64_t)experts * n / 16);
    p.gscale = 1.0f, p.status = status, p.tb = (const uint32_t*)tb, p.off = (const uint32_t*)off, p.row_map = (const uint32_t*)row_map, p.gs = (const float*)gs, p.experts = experts;
    p.msub = mt / 128;
    p.ksplit = 1, p.mpad = 0, p.part = nullptr, p.ldp = 0;
    p.t16b = (const uint8_t*)t16b, p.gsb = (const float*)gsb, p.glu = glu ? 1 : 0, p.limit = limit;
    p.tiles_n = (int)(n / (glu ? kyb::KQ_BN / 2 : kyb::KQ_BN)), p.tiles_m = (int)((s + mt - 1) / mt) + experts;
    p.tma_out = 0, p.col0 = 0, p.wide = 0;                                         // rows are scattered (row_map) or end inside a tile: no tensor map fits
    KybOutMaps outs;
    memset(&outs, 0, sizeof(outs));
    if (int rc = kq_launch(fmt, ta, outs, p, p.tiles_n * p.tiles_m, (cudaStream_t)stream)) return rc;
    return kyb_zero_tail_rows(d, ldd, n, row_map, (const uint32_t*)off + experts, s, (cudaStream_t)stream);   // slots that belong to no expert: rows of zeros
}

extern "C" int kyb_gemm_kq_grouped(int fmt, const void* t16, int64_t n, int64_t k, int experts, const void* a, int64_t lda, int64_t s, const void* tb, const void* off,
                                   const void* row_map, const void* gs, void* d, int64_t ldd, int mt, void* stream) {
    return kq_grouped(fmt, t16, nullptr, n, k, experts, a, lda, s, tb, off, row_map, gs, nullptr, 0.f, d, ldd, mt, stream);
}

// Gate and up of a routed SwiGLU layer as ONE grouped product with the gated activation in its epilogue: h fp16 [s, n] (sorted order) = silu(a) * b with
// a = fp16(x W_gate^T), b = fp16(x W_up^T) (the values the two-launch form would have written) and the optional clamp of kyb_silu_mul. Replaces two
// kyb_gemm_kq_grouped calls and kyb_silu_mul (kyojin_mlx/foreign_kqgmm.py:293-314 `mlp`: gmm, gmm, silu_perm).
extern "C" int kyb_gemm_kq_grouped_glu(int fmt, const void* t16_gate, const void* t16_up, int64_t n, int64_t k, int experts, const void* a, int64_t lda, int64_t s,
                                       const void* tb, const void* off, const void* gs_gate, const void* gs_up, float limit, void* h, int64_t ldh, int mt, void* stream) {
    KYB_REQUIRE(t16_up, "null pointer");
    return kq_grouped(fmt, t16_gate, t16_up, n, k, experts, a, lda, s, tb, off, nullptr, gs_gate, gs_up, limit, h, ldh, mt, stream);
}
