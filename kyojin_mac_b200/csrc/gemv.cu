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
#include <map>
#include <mutex>
#include <tuple>
#include <unordered_map>

#include "t16_decode.cuh"

namespace kyb {

struct GemvParams {
    const uint8_t* t16;
    const __half* x;
    const __half* x2;        // gated input: the staged row is fp16(silu(x row) * x2 row) (same pitch), or null
    __half* y;
    float* partial;          // [nchunks][m][npad]: sums of the canonical k-chunks (form (b))
    unsigned int* status;
    int64_t ldx, ldy;
    int n, npad, nb;         // rows, rows padded to 16, k-blocks of 256
    int m, mst;              // activation rows, rows stored per column tile (1, 2, 4, 8)
    int kbp, ksplit;         // k-blocks per part (cpp chunks), parts
    int kc;                  // k-blocks per canonical chunk: sums are formed per chunk and chunks are added in k order, whatever the split
    int nchunks, cpp;        // canonical chunks along k, chunks per k-part
    int pdl;                 // launched with programmatic stream serialization
    int partial_only;        // every chunk sum goes to `partial` and nothing else is written: form (b), and the two-step entry points with exposed partial sums
    int aligned;             // warps take whole row tiles (no row tile is shared between warps); else runs of whole chunks
    int local;               // form (c): a CTA owns whole row tiles, its warps share their chunks and the chunk sums meet in shared memory (no workspace, no second launch)
    int warps, stages;
    float gscale;
    float limit;             // gated input: > 0 clamps as the activation kernel does
};

constexpr int SCL_STRIDE = 20;                // floats per row of the scale scratch: 16 used; a pitch of 80 bytes lets the 8 row groups of a warp load their 16-byte pieces without bank conflicts
constexpr int SCL_BYTES = 16 * SCL_STRIDE * 4;   // per-warp scale scratch: 16 rows x 16 floats
constexpr int GEMV_STAGES = 2;           // ring depth per warp: a stage is handed back as soon as its tile sits in registers, so two stages keep two copies in flight
constexpr int GEMV_DSTAGES = 2;          // the same for the dense kernel (a four-stage ring measured 1-3 % slower on large matrices: the kernel is not limited by bytes in flight)

template <int FMT>
__host__ __device__ constexpr int xaux_bytes_per_block(int nt) { return kyb_has_mins(FMT) ? 256 * nt : kyb_has_mins16(FMT) ? 512 * nt : 0; }

__device__ __forceinline__ uint32_t magic_sub(uint32_t h2_with_magic, uint32_t sub_bits) {
    __half2 a = *reinterpret_cast<__half2*>(&h2_with_magic), b = *reinterpret_cast<__half2*>(&sub_bits);
    __half2 r = __hsub2(a, b);
    return *reinterpret_cast<uint32_t*>(&r);
}

// ---- per-format: scale preparation (all lanes cooperate, results in scl[16][16] floats) ----------------------------------
template <int FMT>
__device__ __forceinline__ void prep_scales(uint32_t tile, uint32_t scl, int lane) {
    const int r = lane >> 1, hf = lane & 1;
    if constexpr (FMT == KYB_FMT_Q4_K) {
        const uint4 mt = lds128(tile + 2048 + r * 16);
        // 6-bit scales of sub-blocks 4 hf .. 4 hf + 3 as four bytes (kyojin_mlx/foreign_gguf.py:340-346)
        const uint32_t scw = ((hf ? mt.w : mt.y) & (hf ? 0x0f0f0f0fu : 0x3f3f3f3fu)) | ((mt.y >> 2) & (hf ? 0x30303030u : 0u));
        const float d = half_bits_to_float(mt.x & 0xffffu);
        const float dlo = d * 16777216.0f, dhi = d * 1048576.0f;     // the 4-bit codes enter the MMA as fp16 subnormals: even sub-blocks code * 2^-24, odd code * 2^-20
        // byte b -> float without a convert: 0x4B0000bb is 2^23 + b, and fma((2^23 + b), d, -2^23 d) = b d exactly
        const float nlo = dlo * -8388608.0f, nhi = dhi * -8388608.0f;
        float4 o;
        o.x = fmaf(__uint_as_float(prmt(scw, 0x4B000000u, 0x7440u)), dlo, nlo);
        o.y = fmaf(__uint_as_float(prmt(scw, 0x4B000000u, 0x7441u)), dhi, nhi);
        o.z = fmaf(__uint_as_float(prmt(scw, 0x4B000000u, 0x7442u)), dlo, nlo);
        o.w = fmaf(__uint_as_float(prmt(scw, 0x4B000000u, 0x7443u)), dhi, nhi);
        sts128f(scl + 4 * (r * SCL_STRIDE + 4 * hf), o);
    } else if constexpr (FMT == KYB_FMT_Q6_K) {
        const uint2 sw = lds64(tile + 3072 + r * 16 + 8 * hf);
        const float d = half_bits_to_float(lds16(tile + 3328 + r * 2));
        float4 a, b;
        a.x = d * (float)(int)(int8_t)(sw.x & 255u);
        a.y = d * (float)(int)(int8_t)((sw.x >> 8) & 255u);
        a.z = d * (float)(int)(int8_t)((sw.x >> 16) & 255u);
        a.w = d * (float)(int)(int8_t)(sw.x >> 24);
        b.x = d * (float)(int)(int8_t)(sw.y & 255u);
        b.y = d * (float)(int)(int8_t)((sw.y >> 8) & 255u);
        b.z = d * (float)(int)(int8_t)((sw.y >> 16) & 255u);
        b.w = d * (float)(int)(int8_t)(sw.y >> 24);
        sts128f(scl + 4 * (r * SCL_STRIDE + 8 * hf), a);
        sts128f(scl + 4 * (r * SCL_STRIDE + 8 * hf + 4), b);
    } else if constexpr (FMT == KYB_FMT_Q3_K) {
        const uint32_t sp = tile + 1536 + r * 12;
        const uint32_t w0 = lds32(sp), w1 = lds32(sp + 4), w2 = lds32(sp + 8);
        const uint32_t ga = hf ? (((w0 >> 4) & 0x0f0f0f0fu) | (w2 & 0x30303030u)) : ((w0 & 0x0f0f0f0fu) | ((w2 << 4) & 0x30303030u));
        const uint32_t gb = hf ? (((w1 >> 4) & 0x0f0f0f0fu) | ((w2 >> 2) & 0x30303030u)) : ((w1 & 0x0f0f0f0fu) | ((w2 << 2) & 0x30303030u));
        const float d = half_bits_to_float(lds16(tile + 1728 + r * 2));
        float4 a, b;
        a.x = d * (float)((int)(ga & 255u) - 32);
        a.y = d * (float)((int)((ga >> 8) & 255u) - 32);
        a.z = d * (float)((int)((ga >> 16) & 255u) - 32);
        a.w = d * (float)((int)(ga >> 24) - 32);
        b.x = d * (float)((int)(gb & 255u) - 32);
        b.y = d * (float)((int)((gb >> 8) & 255u) - 32);
        b.z = d * (float)((int)((gb >> 16) & 255u) - 32);
        b.w = d * (float)((int)(gb >> 24) - 32);
        sts128f(scl + 4 * (r * SCL_STRIDE + 8 * hf), a);
        sts128f(scl + 4 * (r * SCL_STRIDE + 8 * hf + 4), b);
    } else if constexpr (FMT == KYB_FMT_Q5_K) {
        const uint4 mt = lds128(tile + 2560 + r * 16);
        const uint32_t scw = ((hf ? mt.w : mt.y) & (hf ? 0x0f0f0f0fu : 0x3f3f3f3fu)) | ((mt.y >> 2) & (hf ? 0x30303030u : 0u));   // as Q4_K
        const float d = half_bits_to_float(mt.x & 0xffffu), nd = d * -8388608.0f;                                                  // the 5-bit codes enter the MMA as plain integers
        float4 o;
        o.x = fmaf(__uint_as_float(prmt(scw, 0x4B000000u, 0x7440u)), d, nd);
        o.y = fmaf(__uint_as_float(prmt(scw, 0x4B000000u, 0x7441u)), d, nd);
        o.z = fmaf(__uint_as_float(prmt(scw, 0x4B000000u, 0x7442u)), d, nd);
        o.w = fmaf(__uint_as_float(prmt(scw, 0x4B000000u, 0x7443u)), d, nd);
        sts128f(scl + 4 * (r * SCL_STRIDE + 4 * hf), o);
    } else if constexpr (FMT == KYB_FMT_IQ4_XS) {
        const uint2 mw = lds64(tile + 2048 + r * 8);                       // d | scales_h << 16, four scales_l bytes
        const float d = half_bits_to_float(mw.x & 0xffffu);
        const uint32_t sh = mw.x >> (16 + 8 * hf), sl = mw.y >> (16 * hf);  // sub-blocks 4 hf .. 4 hf + 3: two scales_l bytes, one scales_h byte
        float4 o;
        o.x = d * (float)((int)((sl & 15u) | ((sh & 3u) << 4)) - 32);
        o.y = d * (float)((int)(((sl >> 4) & 15u) | (((sh >> 2) & 3u) << 4)) - 32);
        o.z = d * (float)((int)(((sl >> 8) & 15u) | (((sh >> 4) & 3u) << 4)) - 32);
        o.w = d * (float)((int)(((sl >> 12) & 15u) | (((sh >> 6) & 3u) << 4)) - 32);
        sts128f(scl + 4 * (r * SCL_STRIDE + 4 * hf), o);
    } else if constexpr (FMT == KYB_FMT_Q2_K) {
        const uint2 sw = lds64(tile + 1024 + r * 16 + 8 * hf);             // scale | min << 4 of slices 8 hf .. 8 hf + 7
        const float d = half_bits_to_float(lds16(tile + 1280 + r * 4)) * 16777216.0f;   // the 2-bit codes enter the MMA as fp16 subnormals (code * 2^-24)
        float4 a, b;
        a.x = d * (float)(sw.x & 15u), a.y = d * (float)((sw.x >> 8) & 15u), a.z = d * (float)((sw.x >> 16) & 15u), a.w = d * (float)((sw.x >> 24) & 15u);
        b.x = d * (float)(sw.y & 15u), b.y = d * (float)((sw.y >> 8) & 15u), b.z = d * (float)((sw.y >> 16) & 15u), b.w = d * (float)((sw.y >> 24) & 15u);
        sts128f(scl + 4 * (r * SCL_STRIDE + 8 * hf), a);
        sts128f(scl + 4 * (r * SCL_STRIDE + 8 * hf + 4), b);
    } else if constexpr (FMT == KYB_FMT_Q8_0) {
        const uint2 dw = lds64(tile + 4096 + r * 16 + 8 * hf);             // four of the row's eight fp16 d
        float4 o;
        o.x = half_bits_to_float(dw.x & 0xffffu), o.y = half_bits_to_float(dw.x >> 16), o.z = half_bits_to_float(dw.y & 0xffffu), o.w = half_bits_to_float(dw.y >> 16);
        sts128f(scl + 4 * (r * SCL_STRIDE + 4 * hf), o);
    } else {
        const uint2 sw = lds64(tile + 2048 + r * 16 + 8 * hf);
        float4 a, b;                                                   // e2m1 operands carry 2^-14: fold 2^14 here
        a.x = e4m3_unsigned(sw.x) * 16384.0f;
        a.y = e4m3_unsigned(sw.x >> 8) * 16384.0f;
        a.z = e4m3_unsigned(sw.x >> 16) * 16384.0f;
        a.w = e4m3_unsigned(sw.x >> 24) * 16384.0f;
        b.x = e4m3_unsigned(sw.y) * 16384.0f;
        b.y = e4m3_unsigned(sw.y >> 8) * 16384.0f;
        b.z = e4m3_unsigned(sw.y >> 16) * 16384.0f;
        b.w = e4m3_unsigned(sw.y >> 24) * 16384.0f;
        sts128f(scl + 4 * (r * SCL_STRIDE + 8 * hf), a);
        sts128f(scl + 4 * (r * SCL_STRIDE + 8 * hf + 4), b);
    }
}

template <int NT>
struct Acc {
    float v[NT][4];
};

// ONE: a single activation row is staged (column 0 of the MMA), so the odd accumulator columns are never stored and need no arithmetic
template <int NT, bool ONE>
__device__ __forceinline__ void scale_acc(Acc<NT>& acc, const float (&c)[NT][4], float s_lo, float s_hi) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        acc.v[nt][0] = fmaf(s_lo, c[nt][0], acc.v[nt][0]);
        if (!ONE) acc.v[nt][1] = fmaf(s_lo, c[nt][1], acc.v[nt][1]);
        acc.v[nt][2] = fmaf(s_hi, c[nt][2], acc.v[nt][2]);
        if (!ONE) acc.v[nt][3] = fmaf(s_hi, c[nt][3], acc.v[nt][3]);
    }
}

// ---- the part of a tile one lane keeps in registers, so that the ring stage can be handed back to the copy engine before the arithmetic starts
template <int FMT>
struct TileRegs {
    uint4 q[FMT == KYB_FMT_Q6_K ? 6 : FMT == KYB_FMT_Q3_K ? 3 : FMT == KYB_FMT_Q5_K ? 5 : FMT == KYB_FMT_Q8_0 ? 8 : FMT == KYB_FMT_Q2_K ? 2 : 4];
    uint32_t a0, a1;      // q4_k, q5_k: 6-bit mins of rows g, g + 8 as m16n8k8 A operands; q2_k: 4-bit mins of slices 2t, 2t + 1 (a0, a1) and 2t + 8, 2t + 9 (a2, a3) as m16n8k16 A operands
    uint32_t a2, a3;
    float dmg, dmh;       // q4_k, q5_k: dmin of rows g, g + 8 (scaled to the operand convention)
};

// 6-bit mins of rows g, g + 8 (16 meta bytes per row at `meta`: d, dmin, 12 packed scale / min bytes) as fp16 subnormals (mn * 2^-24) in m16n8k8 A-operand order
template <int FMT>
__device__ __forceinline__ void load_mins(uint32_t meta, int g, int t, TileRegs<FMT>& tr) {
    const uint4 mg = lds128(meta + g * 16), mh = lds128(meta + (g + 8) * 16);
    const bool up = (t & 2) != 0;                  // lanes t = 2, 3 own sub-blocks 4..7
    const uint32_t mka = up ? 0x0f0f0f0fu : 0x3f3f3f3fu, mkb = up ? 0x30303030u : 0u;
    const uint32_t mng = ((up ? mg.w >> 4 : mg.z) & mka) | ((mg.z >> 2) & mkb);
    const uint32_t mnh = ((up ? mh.w >> 4 : mh.z) & mka) | ((mh.z >> 2) & mkb);
    const uint32_t sel = (t & 1) ? 0x4342u : 0x4140u;
    tr.a0 = prmt(mng, 0u, sel), tr.a1 = prmt(mnh, 0u, sel);
    tr.dmg = half_bits_to_float(mg.x >> 16) * 16777216.0f, tr.dmh = half_bits_to_float(mh.x >> 16) * 16777216.0f;
}

template <int FMT>
__device__ __forceinline__ void load_tile(uint32_t tile, int lane, TileRegs<FMT>& tr) {
    const int g = lane >> 2, t = lane & 3;
    if constexpr (FMT == KYB_FMT_Q4_K) {
#pragma unroll
        for (int G = 0; G < 4; ++G) tr.q[G] = lds128(tile + (G * 32 + lane) * 16);
        load_mins<FMT>(tile + 2048, g, t, tr);
    } else if constexpr (FMT == KYB_FMT_Q5_K) {
#pragma unroll
        for (int P = 0; P < 4; ++P) tr.q[P] = lds128(tile + (P * 32 + lane) * 16);
        tr.q[4] = lds128(tile + 2048 + lane * 16);
        load_mins<FMT>(tile + 2560, g, t, tr);
    } else if constexpr (FMT == KYB_FMT_Q8_0) {
#pragma unroll
        for (int P = 0; P < 8; ++P) tr.q[P] = lds128(tile + (P * 32 + lane) * 16);
    } else if constexpr (FMT == KYB_FMT_Q6_K) {
#pragma unroll
        for (int P = 0; P < 4; ++P) tr.q[P] = lds128(tile + (P * 32 + lane) * 16);
        tr.q[4] = lds128(tile + 2048 + lane * 16);
        tr.q[5] = lds128(tile + 2048 + (32 + lane) * 16);
    } else if constexpr (FMT == KYB_FMT_Q2_K) {
        tr.q[0] = lds128(tile + lane * 16);
        tr.q[1] = lds128(tile + (32 + lane) * 16);
        // 4-bit mins (high nibbles of the 16 scale bytes of a row) of slices 2t, 2t + 1 and 2t + 8, 2t + 9 as fp16 subnormals (mn * 2^-24)
        const uint4 sg = lds128(tile + 1024 + g * 16), sh = lds128(tile + 1024 + (g + 8) * 16);
        const uint32_t lo_g = (t & 2) ? sg.y : sg.x, hi_g = (t & 2) ? sg.w : sg.z, lo_h = (t & 2) ? sh.y : sh.x, hi_h = (t & 2) ? sh.w : sh.z;
        const uint32_t sel = (t & 1) ? 0x4342u : 0x4140u;
        tr.a0 = prmt((lo_g >> 4) & 0x0f0f0f0fu, 0u, sel), tr.a1 = prmt((lo_h >> 4) & 0x0f0f0f0fu, 0u, sel);
        tr.a2 = prmt((hi_g >> 4) & 0x0f0f0f0fu, 0u, sel), tr.a3 = prmt((hi_h >> 4) & 0x0f0f0f0fu, 0u, sel);
        tr.dmg = half_bits_to_float(lds16(tile + 1280 + g * 4 + 2)) * 16777216.0f, tr.dmh = half_bits_to_float(lds16(tile + 1280 + (g + 8) * 4 + 2)) * 16777216.0f;
    } else if constexpr (FMT == KYB_FMT_Q3_K) {
        tr.q[0] = lds128(tile + lane * 16);
        tr.q[1] = lds128(tile + (32 + lane) * 16);
        tr.q[2] = lds128(tile + 1024 + lane * 16);
    } else {
#pragma unroll
        for (int P = 0; P < 4; ++P) tr.q[P] = lds128(tile + (P * 32 + lane) * 16);
    }
}

// Sums of the staged activations the minima are multiplied with, as B operands of the correcting MMA (fp16 hi + lo of each fp32 sum). v: 32 inputs (group c2 of
// activation row `row` of column tile nt). Q4_K / Q5_K: one sum per 32 inputs, m16n8k8 order (lane 4 row + j / 2, half j % 2 for sub-block j = c2 % 8; hi at
// word nt * 32 + lane, lo NT * 32 words further). Q2_K: one sum per 16 inputs, m16n8k16 order (slice s: lane 4 row + (s % 8) / 2, register s / 8, half s % 2;
// 8 bytes per lane, hi at (nt * 32 + lane), lo NT * 32 lanes further).
template <int FMT, int NT>
__device__ __forceinline__ void stage_sums(const uint4 (&v)[4], uint8_t* xaux, int c2, int nt, int row) {
    if constexpr (kyb_has_mins(FMT) || kyb_has_mins16(FMT)) {
        float sum[2] = {0.f, 0.f};                                   // one running sum per 32 inputs (element order), or one per 16 inputs
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const __half2* hp = reinterpret_cast<const __half2*>(&v[q]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(hp[e]);
                sum[kyb_has_mins16(FMT) ? (q >> 1) : 0] += f.x + f.y;
            }
        }
        const int blk = c2 >> 3, j = c2 & 7;
        __half* xa = reinterpret_cast<__half*>(xaux + (size_t)blk * xaux_bytes_per_block<FMT>(NT));
        if constexpr (kyb_has_mins(FMT)) {
            const float tot = sum[0];
            const __half hi = __float2half_rn(tot);
            const __half lo = __float2half_rn(tot - __half2float(hi));
            const int idx = (row * 4 + (j >> 1)) * 2 + (j & 1);
            xa[((0 * NT + nt) * 32) * 2 + idx] = hi;
            xa[((1 * NT + nt) * 32) * 2 + idx] = lo;
        } else {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int sl = 2 * j + hf;
                const __half hi = __float2half_rn(sum[hf]);
                const __half lo = __float2half_rn(sum[hf] - __half2float(hi));
                const int idx = ((row * 4 + ((sl & 7) >> 1)) * 2 + (sl >> 3)) * 2 + (sl & 1);
                xa[((0 * NT + nt) * 32) * 4 + idx] = hi;
                xa[((1 * NT + nt) * 32) * 4 + idx] = lo;
            }
        }
    }
}

// ---- one tile (16 rows x 256 inputs) ----------------------------------------------------------------------------------
// xb: this lane's B-fragment pointer for the tile's k-block (chunk c, column tile nt at xb + c * CS + nt * MST * 32, all
// compile-time offsets); xa: this lane's word of the Q4_K sub-block sums of the k-block.
template <int FMT, int NT, int MST>
__device__ __forceinline__ void consume_tile(const TileRegs<FMT>& tr, uint32_t scl, uint32_t xb, uint32_t xa, int lane, Acc<NT>& acc) {
    constexpr int CS = NT * MST * 32;
    const int g = lane >> 2, t = lane & 3;
    auto ldb = [&](int chunk, int nt) -> uint2 { return lds64(xb + chunk * CS + nt * MST * 32); };
    if constexpr (FMT == KYB_FMT_Q4_K) {
        // scales of rows g and g + 8 for the 8 sub-blocks
        const float4 s0a = lds128f(scl + 4 * (g * SCL_STRIDE)), s0b = lds128f(scl + 4 * (g * SCL_STRIDE + 4));
        const float4 s1a = lds128f(scl + 4 * ((g + 8) * SCL_STRIDE)), s1b = lds128f(scl + 4 * ((g + 8) * SCL_STRIDE + 4));
        const float sg[8] = {s0a.x, s0a.y, s0a.z, s0a.w, s0b.x, s0b.y, s0b.z, s0b.w};
        const float sh[8] = {s1a.x, s1a.y, s1a.z, s1a.w, s1b.x, s1b.y, s1b.z, s1b.w};
#pragma unroll
        for (int G = 0; G < 4; ++G) {
            const uint4 u = tr.q[G];
            float clo[NT][4], chi[NT][4];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const uint32_t wg = c ? u.z : u.x, wh = c ? u.w : u.y;
                const uint32_t wg8 = wg >> 8, wh8 = wh >> 8;
                const uint32_t l0 = wg & 0x000F000Fu, l1 = wh & 0x000F000Fu, l2 = wg8 & 0x000F000Fu, l3 = wh8 & 0x000F000Fu;
                const uint32_t h0 = wg & 0x00F000F0u, h1 = wh & 0x00F000F0u, h2 = wg8 & 0x00F000F0u, h3 = wh8 & 0x00F000F0u;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint2 bl = ldb(4 * G + c, nt);
                    const uint2 bh = ldb(4 * G + 2 + c, nt);
                    if (c == 0) {
                        mma16816_z(clo[nt], l0, l1, l2, l3, bl.x, bl.y);
                        mma16816_z(chi[nt], h0, h1, h2, h3, bh.x, bh.y);
                    } else {
                        mma16816(clo[nt], l0, l1, l2, l3, bl.x, bl.y);
                        mma16816(chi[nt], h0, h1, h2, h3, bh.x, bh.y);
                    }
                }
            }
            scale_acc<NT, MST == 1>(acc, clo, sg[2 * G], sh[2 * G]);
            scale_acc<NT, MST == 1>(acc, chi, sg[2 * G + 1], sh[2 * G + 1]);
        }
    } else if constexpr (FMT == KYB_FMT_Q5_K) {
        // scales of rows g and g + 8 for the 8 sub-blocks (d * sc); codes = nibble | fifth bit << 4 as exact fp16 integers
        const float4 s0a = lds128f(scl + 4 * (g * SCL_STRIDE)), s0b = lds128f(scl + 4 * (g * SCL_STRIDE + 4));
        const float4 s1a = lds128f(scl + 4 * ((g + 8) * SCL_STRIDE)), s1b = lds128f(scl + 4 * ((g + 8) * SCL_STRIDE + 4));
        const float sg[8] = {s0a.x, s0a.y, s0a.z, s0a.w, s0b.x, s0b.y, s0b.z, s0b.w};
        const float sh[8] = {s1a.x, s1a.y, s1a.z, s1a.w, s1b.x, s1b.y, s1b.z, s1b.w};
        const uint4 hb = tr.q[4];
#pragma unroll
        for (int P = 0; P < 4; ++P) {
            const uint4 u = tr.q[P];
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {                                         // sub-block j = 2 P + jj = MMA slices 4 P + 2 jj, + 1
                float c[NT][4];
#pragma unroll
                for (int ii = 0; ii < 2; ++ii) {
                    const int s = 4 * P + 2 * jj + ii;
                    uint32_t wg = jj ? u.z : u.x, wh = jj ? u.w : u.y;
                    if (ii) wg >>= 4, wh >>= 4;
                    uint32_t bg = (P & 2) ? hb.z : hb.x, bh = (P & 2) ? hb.w : hb.y;   // word a = s >> 3
                    const int i8 = s & 7;                                               // bit i8 -> bit 4
                    if (i8 < 4) bg <<= (4 - i8), bh <<= (4 - i8);
                    else bg >>= (i8 - 4), bh >>= (i8 - 4);
                    const uint32_t vg = and_or(wg, 0x0F0F0F0Fu, bg & 0x10101010u), vh = and_or(wh, 0x0F0F0F0Fu, bh & 0x10101010u);
                    const uint32_t a0 = magic_sub(prmt(vg, 0x64646464u, 0x4240u), 0x64006400u), a2 = magic_sub(prmt(vg, 0x64646464u, 0x4341u), 0x64006400u);
                    const uint32_t a1 = magic_sub(prmt(vh, 0x64646464u, 0x4240u), 0x64006400u), a3 = magic_sub(prmt(vh, 0x64646464u, 0x4341u), 0x64006400u);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const uint2 b = ldb(s, nt);
                        if (ii == 0) mma16816_z(c[nt], a0, a1, a2, a3, b.x, b.y);
                        else mma16816(c[nt], a0, a1, a2, a3, b.x, b.y);
                    }
                }
                scale_acc<NT, MST == 1>(acc, c, sg[2 * P + jj], sh[2 * P + jj]);
            }
        }
    } else if constexpr (FMT == KYB_FMT_IQ4_XS) {
        // scales of rows g and g + 8 for the 8 sub-blocks (d * (ls - 32)); every 4-bit code is an index into the 16-entry int8 grid: two byte permutes pick
        // the entry from the low and the high half of the table (selector = low 3 bits of four codes at once), bit 3 of each code chooses between them
        const float4 s0a = lds128f(scl + 4 * (g * SCL_STRIDE)), s0b = lds128f(scl + 4 * (g * SCL_STRIDE + 4));
        const float4 s1a = lds128f(scl + 4 * ((g + 8) * SCL_STRIDE)), s1b = lds128f(scl + 4 * ((g + 8) * SCL_STRIDE + 4));
        const float sg[8] = {s0a.x, s0a.y, s0a.z, s0a.w, s0b.x, s0b.y, s0b.z, s0b.w};
        const float sh[8] = {s1a.x, s1a.y, s1a.z, s1a.w, s1b.x, s1b.y, s1b.z, s1b.w};
        auto grid4 = [](uint32_t idx) -> uint32_t {                                   // four codes (one per byte) -> their four grid values + 128 (unsigned bytes)
            const uint32_t x = idx & 0x07070707u, y = x | (x >> 4);
            const uint32_t sel = prmt(y, 0u, 0x4420u);
            const uint32_t lo = prmt(0xBFAD9881u, 0xF6EADDCFu, sel), hi = prmt(0x26190D01u, 0x71594535u, sel);
            const uint32_t m = ((idx >> 3) & 0x01010101u) * 0xFFu;
            return ((lo & ~m) | (hi & m)) ^ 0x80808080u;
        };
#pragma unroll
        for (int P = 0; P < 4; ++P) {
            const uint4 u = tr.q[P];
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {                                         // sub-block 2 P + jj = MMA slices 4 P + 2 jj, + 1
                float c[NT][4];
#pragma unroll
                for (int ii = 0; ii < 2; ++ii) {
                    const int s = 4 * P + 2 * jj + ii;
                    uint32_t wg = jj ? u.z : u.x, wh = jj ? u.w : u.y;
                    if (ii) wg >>= 4, wh >>= 4;
                    const uint32_t vg = grid4(wg & 0x0F0F0F0Fu), vh = grid4(wh & 0x0F0F0F0Fu);
                    // bytes -> fp16 (1024 + v + 128) - 1152 = v, exact
                    const uint32_t a0 = magic_sub(prmt(vg, 0x64646464u, 0x4240u), 0x64806480u), a2 = magic_sub(prmt(vg, 0x64646464u, 0x4341u), 0x64806480u);
                    const uint32_t a1 = magic_sub(prmt(vh, 0x64646464u, 0x4240u), 0x64806480u), a3 = magic_sub(prmt(vh, 0x64646464u, 0x4341u), 0x64806480u);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const uint2 b = ldb(s, nt);
                        if (ii == 0) mma16816_z(c[nt], a0, a1, a2, a3, b.x, b.y);
                        else mma16816(c[nt], a0, a1, a2, a3, b.x, b.y);
                    }
                }
                scale_acc<NT, MST == 1>(acc, c, sg[2 * P + jj], sh[2 * P + jj]);
            }
        }
    } else if constexpr (FMT == KYB_FMT_Q8_0) {
#pragma unroll
        for (int P = 0; P < 8; ++P) {                                                // block P of 32 inputs = MMA slices 2 P, 2 P + 1, one fp16 d
            const uint4 u = tr.q[P];
            const float sgv = __uint_as_float(lds32(scl + 4 * (g * SCL_STRIDE + P))), shv = __uint_as_float(lds32(scl + 4 * ((g + 8) * SCL_STRIDE + P)));
            float c[NT][4];
#pragma unroll
            for (int p2 = 0; p2 < 2; ++p2) {
                const uint32_t vg = (p2 ? u.z : u.x) ^ 0x80808080u, vh = (p2 ? u.w : u.y) ^ 0x80808080u;   // int8 -> value + 128
                // bytes -> fp16 (1024 + v + 128) - 1152 = v, exact
                const uint32_t a0 = magic_sub(prmt(vg, 0x64646464u, 0x4240u), 0x64806480u), a2 = magic_sub(prmt(vg, 0x64646464u, 0x4341u), 0x64806480u);
                const uint32_t a1 = magic_sub(prmt(vh, 0x64646464u, 0x4240u), 0x64806480u), a3 = magic_sub(prmt(vh, 0x64646464u, 0x4341u), 0x64806480u);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint2 b = ldb(2 * P + p2, nt);
                    if (p2 == 0) mma16816_z(c[nt], a0, a1, a2, a3, b.x, b.y);
                    else mma16816(c[nt], a0, a1, a2, a3, b.x, b.y);
                }
            }
            scale_acc<NT, MST == 1>(acc, c, sgv, shv);
        }
    } else {
        uint4 hi = make_uint4(0, 0, 0, 0), hb = make_uint4(0, 0, 0, 0);
        if constexpr (FMT == KYB_FMT_Q3_K) hb = tr.q[2];
#pragma unroll
        for (int P = 0; P < 4; ++P) {
            // one scale per MMA slice s = 4 P + i
            const float4 sg4 = lds128f(scl + 4 * (g * SCL_STRIDE + 4 * P)), sh4 = lds128f(scl + 4 * ((g + 8) * SCL_STRIDE + 4 * P));
            const float sg[4] = {sg4.x, sg4.y, sg4.z, sg4.w}, sh[4] = {sh4.x, sh4.y, sh4.z, sh4.w};
            uint4 u;
            if constexpr (FMT == KYB_FMT_Q6_K) {
                u = tr.q[P];
                hi = tr.q[4 + (P >> 1)];
            } else if constexpr (FMT == KYB_FMT_Q3_K || FMT == KYB_FMT_Q2_K) {
                hi = tr.q[P >> 1];                                                       // 2-bit plane
                u = hi;
            } else {
                u = tr.q[P];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
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
                } else if constexpr (FMT == KYB_FMT_Q2_K) {
                    uint32_t wg = (P & 1) ? u.z : u.x, wh = (P & 1) ? u.w : u.y;     // word a = (s >> 2) & 1 = P & 1
                    wg = (wg >> (2 * i)) & 0x03030303u, wh = (wh >> (2 * i)) & 0x03030303u;
                    // a byte in a 16-bit lane is the fp16 subnormal code * 2^-24: exact, and the 2^24 sits in the block scale
                    a0 = prmt(wg, 0u, 0x4240u), a2 = prmt(wg, 0u, 0x4341u);
                    a1 = prmt(wh, 0u, 0x4240u), a3 = prmt(wh, 0u, 0x4341u);
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
                    const uint2 b = ldb(s, nt);
                    mma16816_z(c[nt], a0, a1, a2, a3, b.x, b.y);
                }
                scale_acc<NT, MST == 1>(acc, c, sg[i], sh[i]);
            }
        }
    }
    if constexpr (kyb_has_mins(FMT)) {
        // minus dmin * sum_j mn_j * (sum of x over sub-block j): an m16n8k8 product of the 6-bit mins with the staged sums (fp16 hi + lo)
        const uint32_t a0 = tr.a0, a1 = tr.a1;
        const float dmg = tr.dmg, dmh = tr.dmh;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float tt[4];
            mma1688_z(tt, a0, a1, lds32(xa + (0 * NT + nt) * 128));
            mma1688(tt, a0, a1, lds32(xa + (1 * NT + nt) * 128));
            acc.v[nt][0] = fmaf(-dmg, tt[0], acc.v[nt][0]);
            if (MST != 1) acc.v[nt][1] = fmaf(-dmg, tt[1], acc.v[nt][1]);
            acc.v[nt][2] = fmaf(-dmh, tt[2], acc.v[nt][2]);
            if (MST != 1) acc.v[nt][3] = fmaf(-dmh, tt[3], acc.v[nt][3]);
        }
    }
    if constexpr (kyb_has_mins16(FMT)) {
        // minus dmin * sum_s mn_s * (sum of x over slice s): one m16n8k16 product of the 4-bit mins with the staged per-slice sums (fp16 hi + lo)
        const float dmg = tr.dmg, dmh = tr.dmh;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float tt[4];
            const uint2 bh = lds64(xa + (0 * NT + nt) * 256), bl = lds64(xa + (1 * NT + nt) * 256);
            mma16816_z(tt, tr.a0, tr.a1, tr.a2, tr.a3, bh.x, bh.y);
            mma16816(tt, tr.a0, tr.a1, tr.a2, tr.a3, bl.x, bl.y);
            acc.v[nt][0] = fmaf(-dmg, tt[0], acc.v[nt][0]);
            if (MST != 1) acc.v[nt][1] = fmaf(-dmg, tt[1], acc.v[nt][1]);
            acc.v[nt][2] = fmaf(-dmh, tt[2], acc.v[nt][2]);
            if (MST != 1) acc.v[nt][3] = fmaf(-dmh, tt[3], acc.v[nt][3]);
        }
    }
}

// fp16(silu(a) * b) on 8 values, the arithmetic of silu_mul_kernel (fp32, saturated)
__device__ __forceinline__ uint4 glu8(const uint4 a, const uint4 b, const float limit) {
    const __half* ah = reinterpret_cast<const __half*>(&a);
    const __half* bh = reinterpret_cast<const __half*>(&b);
    uint4 o;
    __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float av = __half2float(ah[j]), bv = __half2float(bh[j]);
        if (limit > 0.f) av = fminf(av, limit), bv = fminf(fmaxf(bv, -limit), limit);
        oh[j] = sat_half(av * (1.0f / (1.0f + expf(-av))) * bv);
    }
    return o;
}

// Single CTA: slots -> groups. counts per expert, groups per expert = ceil(count / 8), slot p of rank r inside its expert -> group start + r / 8.
__global__ void moe_groups_kernel(const uint32_t* __restrict__ eids, int S, int E, uint32_t* __restrict__ g_expert, uint32_t* __restrict__ g_slots, uint32_t* __restrict__ ngroups) {
    extern __shared__ uint32_t gsm[];
    uint32_t* counts = gsm;          // [E]
    uint32_t* gstart = gsm + E;      // [E + 1]
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0u;
    for (int i = threadIdx.x; i < S * 8; i += blockDim.x) g_slots[i] = 0xFFFFFFFFu;
    __syncthreads();
    for (int p = threadIdx.x; p < S; p += blockDim.x)
        if (eids[p] < (uint32_t)E) atomicAdd(&counts[eids[p]], 1u);
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t g = 0;
        for (int e = 0; e < E; ++e) {
            gstart[e] = g;
            g += (counts[e] + 7u) >> 3;
        }
        gstart[E] = g;
        *ngroups = g;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        for (uint32_t g = gstart[e]; g < gstart[e + 1]; ++g) g_expert[g] = (uint32_t)e;
        counts[e] = 0u;                                   // reused as the rank cursor
    }
    __syncthreads();
    for (int p = threadIdx.x; p < S; p += blockDim.x) {
        const uint32_t e = eids[p];
        if (e >= (uint32_t)E) continue;
        const uint32_t r = atomicAdd(&counts[e], 1u);
        g_slots[(size_t)(gstart[e] + (r >> 3)) * 8 + (r & 7u)] = (uint32_t)p;
    }
}

// Persistent kernel, one CTA per SM. The work of a matrix is cut into UNITS: (16-row tile, canonical k-chunk of kc k-blocks); units are ordered row tile by
// row tile, which is also their order in memory. CTA c works on k-part c % ksplit (it stages the activations of that part once); the units of a part are dealt
// to the warps of its CTAs as contiguous, equally long runs, so every warp streams one contiguous range of tiles and all warps finish together. A warp forms the
// sum of every chunk in registers. Three forms: (a) matrices with many row tiles: a run is whole row tiles, the warp adds the chunk sums in k order and stores y
// itself; (b) otherwise a run is whole chunks (+-1 over the warps whatever the shape), every chunk sum goes to the workspace and gemv_finalize_kernel adds them in
// k order; (c) small matrices, where a second launch would cost as much as the product: CTA c owns the row tiles [ntiles c / G, ntiles (c + 1) / G), its warps
// share the chunks of those row tiles as in (b), the chunk sums go to shared memory and after a CTA barrier the threads add them in k order and store y.
// Either way an output is the left-to-right sum of the same chunk sums, so results do not depend on the batch size, the grid or the split.
template <int FMT, int NT, int MST>
// At most 16 warps per CTA: 128 registers per thread let the compiler keep the unpacked operands of several MMAs in flight (with 24 warps and 80 registers the
// kernel spilled and its steady rate was 15 % lower).
__global__ void __launch_bounds__(NT <= 2 ? 512 : 256, 1) gemv_t16_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int TB = kyb_tile_bytes(FMT);
    constexpr int CS = NT * MST * 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kp = blockIdx.x % p.ksplit, cgi = blockIdx.x / p.ksplit;
    const int c0 = kp * p.cpp, cpk = min(p.nchunks, c0 + p.cpp) - c0;             // first chunk and number of chunks of this k-part
    const int kb0 = c0 * p.kc, nblk = min(p.nb, (c0 + cpk) * p.kc) - kb0;         // its k-blocks
    const int part_ctas = ((int)gridDim.x - kp + p.ksplit - 1) / p.ksplit;        // CTAs working on this k-part
    const int WP = part_ctas * p.warps, ws = cgi * p.warps + warp;
    const int ntiles = p.npad >> 4;
    const int64_t UP = (int64_t)ntiles * cpk;                                     // units of this part
    // this warp's run: whole row tiles when the plan says so (many row tiles: no row tile is shared, nothing goes through the workspace), else whole chunks
    const bool local = p.local != 0;                                              // form (c): one k-part, cpk = nchunks
    const int rtA = local ? (int)((int64_t)ntiles * blockIdx.x / gridDim.x) : 0, rtB = local ? (int)((int64_t)ntiles * (blockIdx.x + 1) / gridDim.x) : 0;
    const int64_t UL = (int64_t)(rtB - rtA) * cpk;                                // units of this CTA's row tiles
    const int64_t u0 = local       ? (int64_t)rtA * cpk + UL * warp / p.warps
                       : p.aligned ? (int64_t)ntiles * ws / WP * cpk
                                   : UP * ws / WP,
                  u1 = local       ? (int64_t)rtA * cpk + UL * (warp + 1) / p.warps
                       : p.aligned ? (int64_t)ntiles * (ws + 1) / WP * cpk
                                   : UP * (ws + 1) / WP;
    auto tiles_before = [&](int64_t u) -> int64_t { return (u / cpk) * nblk + (u % cpk) * p.kc; };
    const int total = (int)(tiles_before(u1) - tiles_before(u0));
    const int rt0 = (int)(u0 / cpk), j0 = (int)(u0 % cpk);

    // ---- shared memory carve-up
    uint8_t* xfrag = smem;
    uint8_t* xaux = xfrag + (size_t)p.kbp * 16 * CS;
    constexpr int STAGES = GEMV_DSTAGES;
    constexpr size_t warp_bytes = ((size_t)STAGES * TB + SCL_BYTES + 8 * (size_t)STAGES + 8 + 15) & ~(size_t)15;
    uint8_t* wbase = xaux + (size_t)p.kbp * xaux_bytes_per_block<FMT>(NT) + (size_t)warp * warp_bytes;
    uint8_t* ring = wbase;
    float* scl = reinterpret_cast<float*>(wbase + (size_t)STAGES * TB);
    uint64_t* bars = reinterpret_cast<uint64_t*>(wbase + (size_t)STAGES * TB + SCL_BYTES);
    float* cpart = reinterpret_cast<float*>(xaux + (size_t)p.kbp * xaux_bytes_per_block<FMT>(NT) + (size_t)p.warps * warp_bytes);   // form (c): [row tile][chunk][m][16 rows]

    // producer state (lane 0): next tile to request. The tiles of a row tile's part are contiguous; the next row tile follows nb - nblk tiles further.
    int p_left = total, p_blk = nblk - j0 * p.kc;             // tiles still to request, tiles left in the current row tile's part
    const uint8_t* p_src = p.t16 + ((size_t)rt0 * (size_t)p.nb + (size_t)(kb0 + j0 * p.kc)) * TB;
    const size_t p_jump = (size_t)(p.nb - nblk) * TB;
    const uint32_t ring_a = smem_u32(ring), bar_a = smem_u32(bars), scl_a = smem_u32(scl);
    auto issue = [&](int stage) {
        const uint32_t bar = bar_a + 8 * stage, dst = ring_a + stage * TB;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)TB) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(p_src), "r"((uint32_t)TB), "r"(bar)
                     : "memory");
        --p_left;
        p_src += TB;
        if (--p_blk == 0) p_blk = nblk, p_src += p_jump;
    };

    // ---- start the weight stream before staging x: the copies run while the CTA prepares the activations
    if (p.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // a dependent launch may start its own weight prefetch as SMs free up
    if (lane == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(&bars[s], 1);
        mbar_fence_init();
        const int pre = min(STAGES, total);
        for (int s = 0; s < pre; ++s) issue(s);
    }
    // weights are never written by a preceding kernel, activations and outputs may be: everything below waits for the launch this one depends on
    if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- stage activations of this k-part as B fragments: [chunk][nt][row < MST][lane t][4 halves permuted (0, 2, 1, 3)].
    // One item = 32 inputs of one activation row (two chunks = one Q4_K sub-block); q4_k also gets the sum of the 32 inputs, split into
    // fp16 hi + lo and laid out as m16n8k8 B fragments (lane 4 g + t: sub-blocks 2t, 2t + 1 of row g).
    {
        const int items = nblk * 8 * NT * MST;
        constexpr int U = 4;                                   // loads of U items are in flight together (x comes from L2)
        for (int it0 = threadIdx.x; it0 < items; it0 += U * blockDim.x) {
            uint4 v[U][4];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int it = it0 + u * blockDim.x;
#pragma unroll
                for (int q = 0; q < 4; ++q) v[u][q] = make_uint4(0, 0, 0, 0);
                if (it < items) {
                    const int row = it % MST, nt = (it / MST) % NT, c2 = it / (MST * NT);
                    const int m = nt * 8 + row;
                    if (m < p.m) {
                        const uint4* xp = reinterpret_cast<const uint4*>(p.x + (size_t)m * p.ldx + (size_t)kb0 * 256 + (size_t)c2 * 32);
#pragma unroll
                        for (int q = 0; q < 4; ++q) v[u][q] = __ldg(xp + q);
                        if (p.x2) {                                          // gated input: the activation is formed while the row is staged
                            const uint4* xq = reinterpret_cast<const uint4*>(p.x2 + (size_t)m * p.ldx + (size_t)kb0 * 256 + (size_t)c2 * 32);
#pragma unroll
                            for (int q = 0; q < 4; ++q) v[u][q] = glu8(v[u][q], __ldg(xq + q), p.limit);
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int it = it0 + u * blockDim.x;
                if (it < items) {
                    const int row = it % MST, nt = (it / MST) % NT, c2 = it / (MST * NT);
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const uint4 a = v[u][2 * c], b = v[u][2 * c + 1];
                        uint4 oa, ob;
                        oa.x = prmt(a.x, a.y, 0x5410u), oa.y = prmt(a.x, a.y, 0x7632u), oa.z = prmt(a.z, a.w, 0x5410u), oa.w = prmt(a.z, a.w, 0x7632u);
                        ob.x = prmt(b.x, b.y, 0x5410u), ob.y = prmt(b.x, b.y, 0x7632u), ob.z = prmt(b.z, b.w, 0x5410u), ob.w = prmt(b.z, b.w, 0x7632u);
                        uint4* dst = reinterpret_cast<uint4*>(xfrag + (size_t)(2 * c2 + c) * CS + (nt * MST + row) * 32);
                        dst[0] = oa, dst[1] = ob;
                    }
                    stage_sums<FMT, NT>(v[u], xaux, c2, nt, row);
                }
            }
        }
    }
    __syncthreads();
    if (total == 0 && !local) return;

    const int g = lane >> 2, t = lane & 3;
    // lanes whose activation row is not staged read a staged row instead: their output columns are never stored
    const uint32_t xb0 = smem_u32(xfrag) + (g & (MST - 1)) * 32 + t * 8, xa0 = smem_u32(xaux) + lane * (kyb_has_mins16(FMT) ? 8 : 4);
    uint32_t xb = xb0 + (uint32_t)(j0 * p.kc) * (16 * CS), xa = xa0 + (uint32_t)(j0 * p.kc) * xaux_bytes_per_block<FMT>(NT);   // this lane's fragment addresses for the current k-block

    Acc<NT> acc, tot;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc.v[nt][q] = 0.f, tot.v[nt][q] = 0.f;
    const bool whole = !p.partial_only;                           // every row tile of the run is complete (whole row tiles per warp, one k-part)
    int rt = rt0, j = j0, cleft = min(p.kc, nblk - j0 * p.kc);
    uint32_t parity = 0;
    bool failed = false;
    auto step = [&](const int stage) {                            // stage is a literal at every call: all shared addresses are base + immediate
        const uint32_t tile = ring_a + stage * TB;
        // a wait that gives up is remembered; the tile is then consumed as it is (its values do not matter any more) and the kernel reports at the end
        if (!mbar_wait_fast(bar_a + 8 * stage, parity)) failed = true;
        // phase A: everything this warp needs from the stage goes to registers / the scale scratch, then the stage is handed back and refilled
        TileRegs<FMT> tr;
        load_tile<FMT>(tile, lane, tr);
        prep_scales<FMT>(tile, scl_a, lane);
        __syncwarp();
        if (lane == 0 && p_left > 0) issue(stage);
        // phase B: arithmetic from registers
        consume_tile<FMT, NT, MST>(tr, scl_a, xb, xa, lane, acc);
        __syncwarp();                                             // the scale scratch is rewritten by the next tile
        xb += 16 * CS, xa += xaux_bytes_per_block<FMT>(NT);
        if (--cleft == 0) {
            // ---- end of a canonical chunk. lane (g, t) holds rows g, g + 8 x activation rows 2t, 2t + 1 of each column tile
            const int chunk = c0 + j;
            const bool rt_done = ++j == cpk;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int nrow = rt * 16 + g + 8 * (q >> 1), m = nt * 8 + 2 * t + (q & 1);
                    if (whole) {
                        tot.v[nt][q] += acc.v[nt][q];
                        if (rt_done) {
                            if (m < p.m && nrow < p.n) p.y[(size_t)m * p.ldy + nrow] = sat_half(tot.v[nt][q] * p.gscale);
                            tot.v[nt][q] = 0.f;
                        }
                    } else if (m < p.m) {
                        if (local) cpart[((size_t)((rt - rtA) * cpk + chunk) * p.m + m) * 16 + g + 8 * (q >> 1)] = acc.v[nt][q];
                        else p.partial[((size_t)chunk * p.m + m) * p.npad + nrow] = acc.v[nt][q];
                    }
                    acc.v[nt][q] = 0.f;
                }
            }
            if (rt_done) j = 0, ++rt, xb = xb0, xa = xa0;
            cleft = min(p.kc, nblk - j * p.kc);
        }
    };
    static_assert(STAGES == 2, "the tile loop alternates the stages of a two-stage ring");
    int i = 0;
    for (; i + 1 < total; i += 2) {
        step(0);
        step(1);
        parity ^= 1u;
    }
    if (i < total) step(0);
    // every requested tile was waited for above (bounded), so no copy of this warp is in flight here
    if (__any_sync(0xffffffffu, failed) && lane == 0) atomicExch(p.status, KYB_DEV_TIMEOUT_GEMV);
    if (local) {
        // form (c): the chunk sums of this CTA's row tiles are added in k order, as the finalize kernel of form (b) adds them
        __syncthreads();
        const int outs = (rtB - rtA) * 16 * p.m;
        for (int i = threadIdx.x; i < outs; i += blockDim.x) {
            const int row = i & 15, m = (i >> 4) % p.m, rtl = (i >> 4) / p.m, nrow = (rtA + rtl) * 16 + row;
            float s = 0.f;
            for (int c = 0; c < cpk; ++c) s += cpart[((size_t)(rtl * cpk + c) * p.m + m) * 16 + row];
            if (nrow < p.n) p.y[(size_t)m * p.ldy + nrow] = sat_half(s * p.gscale);
        }
    }
}

// ------------------------------------------------------------------------------------------------ routed experts: grouped GEMV with expert election
// Slots routed to the same expert are served together: group = (expert, up to 8 of its slots), so an expert's bytes are read once per 8 slots
// (the reference's `moe_union` election, kyojin_mlx/moe_union.py:27-63, done for 8 rows because the MMA has 8 activation columns anyway).
struct GroupParams {
    const uint8_t* t16;            // expert stack: E matrices of n rows
    const uint8_t* t16b;           // pair form: a second stack of the same shape served by the same launch (its results are rows [S, 2 S) of y), or null
    const __half* x;               // [*, k] source rows
    const __half* x2;              // gated form: the staged row is fp16(silu(x row) * x2 row) (same row index, same pitch), or null
    const uint32_t* eids;          // [S] expert of each slot, or null; rows of slots whose id is outside [0, E) are set to zero
    const uint32_t* xrows;         // [S] source row of each slot, or null (slot s reads row s / xdiv)
    const uint32_t* g_expert;      // [G]
    const uint32_t* g_slots;       // [G * 8] slot or 0xFFFFFFFF
    const uint32_t* ngroups;       // device scalar
    const float* gs;               // per-expert output scale or null
    const float* gsb;              // the same for the second stack
    __half* y;                     // [S, ldy] ([2 S, ldy] in the pair form)
    unsigned int* status;
    int64_t ldx, ldy;
    float limit;                   // gated form: > 0 clamps as the activation kernel does
    int n, nb, kc, xdiv, rc, warps;   // rows per expert, k-blocks, canonical chunk, slot -> row divisor, row chunks per group, warps per CTA
    int S, E;
};

template <int FMT>
// at most 16 warps: 128 registers per thread (with 24 warps and 80 registers the same layer ran 14 % slower, with 20 warps 5 %)
__global__ void __launch_bounds__(512, 1) gemv_group_kernel(const GroupParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int TB = kyb_tile_bytes(FMT), NT = 1, MST = 8, CS = NT * MST * 32, STAGES = GEMV_STAGES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    uint8_t* xfrag = smem;
    uint8_t* xaux = xfrag + (size_t)p.nb * 16 * CS;
    constexpr size_t warp_bytes = ((size_t)STAGES * TB + SCL_BYTES + 8 * (size_t)STAGES + 8 + 15) & ~(size_t)15;
    uint8_t* wbase = xaux + (size_t)p.nb * xaux_bytes_per_block<FMT>(NT) + (size_t)warp * warp_bytes;
    const uint32_t ring_a = smem_u32(wbase), scl_a = ring_a + STAGES * TB, bar_a = scl_a + SCL_BYTES;
    __shared__ uint32_t s_slots[8];
    if (lane == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init_a_local(bar_a + 8 * s);
        mbar_fence_init();
    }
    __syncthreads();
    const int ntiles = p.n >> 4;                                   // row tiles per expert (n % 16 == 0)
    const int tpc = (ntiles + p.rc - 1) / p.rc;                    // row tiles per chunk
    const uint32_t ngroups = *p.ngroups;
    const uint32_t xb0 = smem_u32(xfrag) + g * 32 + t * 8, xa0 = smem_u32(xaux) + lane * (kyb_has_mins16(FMT) ? 8 : 4);
    const uint32_t npair = p.t16b ? 2u : 1u;
    // slots that belong to no expert are in no group: their rows are written here
    if (p.eids)
        for (int sl = blockIdx.x; sl < p.S; sl += gridDim.x)
            if (p.eids[sl] >= (uint32_t)p.E)
                for (uint32_t w2 = 0; w2 < npair; ++w2)
                    for (int c = threadIdx.x; c < p.n; c += blockDim.x) p.y[((size_t)sl + (size_t)w2 * p.S) * p.ldy + c] = __float2half(0.f);
    uint32_t parity = 0;
    int stage = 0;
    bool failed = false;
    // Items go to the CTAs round-robin and all cost the same, so the last round would keep only `rest` of the CTAs busy for a whole item (904 items on 148 CTAs:
    // six full rounds and a seventh for 16 of them). The items of that last round are therefore cut into `cut` parts of their row tiles each (as many as there are
    // idle CTAs per item, while every warp still gets a row tile): the round then lasts 1 / cut of an item. A row tile is still computed by one warp over the whole
    // of k, so no result changes.
    const uint32_t whole_items = ngroups * (uint32_t)p.rc * npair;
    const uint32_t even = whole_items / gridDim.x * gridDim.x, rest = whole_items - even;
    const uint32_t cut = rest ? max(1u, min(gridDim.x / rest, (uint32_t)max(1, tpc / p.warps))) : 1u;
    for (uint32_t item = blockIdx.x; item < even + rest * cut; item += gridDim.x) {
        const uint32_t whole = item < even ? item : even + (item - even) / cut, part = item < even ? 0u : (item - even) % cut, parts = item < even ? 1u : cut;
        const uint32_t which = whole % npair, it2 = whole / npair;            // the two stacks of a pair take neighbouring items
        const uint32_t grp = it2 / (uint32_t)p.rc, rc = it2 % (uint32_t)p.rc;
        const uint32_t e = p.g_expert[grp];
        const uint8_t* stack = which ? p.t16b : p.t16;
        const int c_begin = (int)rc * tpc, c_len = max(0, min(ntiles, ((int)rc + 1) * tpc) - c_begin);
        const int rt0 = c_begin + (int)((uint32_t)c_len * part / parts) + warp, rt_end = c_begin + (int)((uint32_t)c_len * (part + 1) / parts);
        const int nrt = rt0 < rt_end ? (rt_end - rt0 + p.warps - 1) / p.warps : 0;      // row tiles of this warp: rt0, rt0 + warps, ...
        const int total = nrt * p.nb;
        // ---- producer (lane 0): this item's tiles of this warp
        int p_left = total, p_blk = p.nb, p_stage = stage;
        const uint8_t* p_src = stack + (((size_t)e * ntiles + rt0) * (size_t)p.nb) * TB;
        const size_t p_jump = ((size_t)p.warps - 1) * (size_t)p.nb * TB;
        auto issue = [&]() {
            const uint32_t bar = bar_a + 8 * p_stage, dst = ring_a + p_stage * TB;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)TB) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(p_src), "r"((uint32_t)TB), "r"(bar) : "memory");
            --p_left;
            p_src += TB;
            if (--p_blk == 0) p_blk = p.nb, p_src += p_jump;
            p_stage ^= 1;
        };
        if (lane == 0)
            for (int s = 0; s < min(STAGES, total); ++s) issue();
        if (threadIdx.x < 8) s_slots[threadIdx.x] = p.g_slots[(size_t)grp * 8 + threadIdx.x];
        __syncthreads();
        // ---- stage the group's activation rows (gathered) as B fragments, as in gemv_t16_kernel
        {
            const int items = p.nb * 8 * MST;
            for (int it = threadIdx.x; it < items; it += blockDim.x) {
                const int row = it % MST, c2 = it / MST;
                const uint32_t slot = s_slots[row];
                uint4 v[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) v[q] = make_uint4(0, 0, 0, 0);
                if (slot != 0xFFFFFFFFu) {
                    const size_t xr = p.xrows ? p.xrows[slot] : slot / (uint32_t)p.xdiv;
                    const uint4* xp = reinterpret_cast<const uint4*>(p.x + xr * p.ldx + (size_t)c2 * 32);
#pragma unroll
                    for (int q = 0; q < 4; ++q) v[q] = __ldg(xp + q);
                    if (p.x2) {                                               // gated input: the activation is formed while the row is staged
                        const uint4* xq = reinterpret_cast<const uint4*>(p.x2 + xr * p.ldx + (size_t)c2 * 32);
#pragma unroll
                        for (int q = 0; q < 4; ++q) v[q] = glu8(v[q], __ldg(xq + q), p.limit);
                    }
                }
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const uint4 a = v[2 * c], b = v[2 * c + 1];
                    uint4 oa, ob;
                    oa.x = prmt(a.x, a.y, 0x5410u), oa.y = prmt(a.x, a.y, 0x7632u), oa.z = prmt(a.z, a.w, 0x5410u), oa.w = prmt(a.z, a.w, 0x7632u);
                    ob.x = prmt(b.x, b.y, 0x5410u), ob.y = prmt(b.x, b.y, 0x7632u), ob.z = prmt(b.z, b.w, 0x5410u), ob.w = prmt(b.z, b.w, 0x7632u);
                    uint4* dst = reinterpret_cast<uint4*>(xfrag + (size_t)(2 * c2 + c) * CS + row * 32);
                    dst[0] = oa, dst[1] = ob;
                }
                stage_sums<FMT, NT>(v, xaux, c2, 0, row);
            }
        }
        __syncthreads();
        // ---- this warp's row tiles
        Acc<NT> acc, tot;
#pragma unroll
        for (int q = 0; q < 4; ++q) acc.v[0][q] = 0.f, tot.v[0][q] = 0.f;
        const float* gsp = which ? p.gsb : p.gs;
        const float gsc = gsp ? gsp[e] : 1.0f;
        const size_t yrow0 = which ? (size_t)p.S : 0;
        uint32_t xb = xb0, xa = xa0;
        int blk = 0, rt = rt0, cleft = min(p.kc, p.nb);
        for (int i = 0; i < total; ++i) {
            const uint32_t tile = ring_a + stage * TB;
            if (!mbar_wait_fast(bar_a + 8 * stage, parity)) failed = true;
            TileRegs<FMT> tr;
            load_tile<FMT>(tile, lane, tr);
            prep_scales<FMT>(tile, scl_a, lane);
            __syncwarp();
            if (lane == 0 && p_left > 0) issue();
            consume_tile<FMT, NT, MST>(tr, scl_a, xb, xa, lane, acc);
            __syncwarp();
            xb += 16 * CS, xa += xaux_bytes_per_block<FMT>(NT);
            ++blk;
            if (--cleft == 0) {
                const bool last = blk == p.nb;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    tot.v[0][q] += acc.v[0][q];
                    acc.v[0][q] = 0.f;
                    if (last) {
                        const uint32_t slot = s_slots[2 * t + (q & 1)];
                        const int nrow = rt * 16 + g + 8 * (q >> 1);
                        if (slot != 0xFFFFFFFFu) p.y[(yrow0 + slot) * p.ldy + nrow] = sat_half(tot.v[0][q] * gsc);
                        tot.v[0][q] = 0.f;
                    }
                }
                cleft = min(p.kc, p.nb - blk);
                if (last) blk = 0, rt += p.warps, xb = xb0, xa = xa0, cleft = min(p.kc, p.nb);
            }
            stage ^= 1;
            if (stage == 0) parity ^= 1u;
        }
        __syncthreads();                                          // the staged rows are replaced by the next item
    }
    if (__any_sync(0xffffffffu, failed) && lane == 0) atomicExch(p.status, KYB_DEV_TIMEOUT_GEMV);
}

__global__ void gemv_finalize_kernel(const float* __restrict__ partial, int ksplit, int m, int n, int npad, float gscale, __half* __restrict__ y, int64_t ldy) {
    // in a chained launch the CTAs of this kernel may be resident while the GEMV's last warps finish, and the next kernel of the chain may start its own
    // weight prefetch at once: the partial sums are complete and visible after the wait; both instructions are no-ops under a plain launch
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)m * n) return;
    const int row = (int)(i / n), col = (int)(i % n);
    float s = 0.f;
    for (int c = 0; c < ksplit; ++c) s += partial[((size_t)c * m + row) * npad + col];     // ksplit = number of canonical chunks here
    y[(size_t)row * ldy + col] = sat_half(s * gscale);
}

}  // namespace kyb

// ------------------------------------------------------------------------------------------------ host side
namespace {

struct GemvPlan {
    int nt, mst, warps, stages, kbp, ksplit, grid;
    size_t smem;
    int kc, nchunks, cpp, aligned;
    int local;
};

size_t plan_smem(int fmt, int nt, int mst, int kbp, int warps, int stages) {
    const size_t tb = kyb_tile_bytes(fmt);
    const size_t xfrag = (size_t)kbp * 16 * nt * mst * 32;
    const size_t xaux = kyb_has_mins(fmt) ? (size_t)kbp * 256 * nt : kyb_has_mins16(fmt) ? (size_t)kbp * 512 * nt : 0;
    const size_t wb = ((size_t)stages * tb + kyb::SCL_BYTES + 8 * (size_t)stages + 8 + 15) & ~(size_t)15;
    return xfrag + xaux + warps * wb;
}

// kernel variants: (column tiles, staged activation rows per tile)
constexpr int NVAR = 6;
constexpr int VAR_NT[NVAR] = {1, 1, 1, 1, 2, 4}, VAR_MST[NVAR] = {1, 2, 4, 8, 8, 8};

int variant_of(int64_t m) { return m <= 1 ? 0 : m <= 2 ? 1 : m <= 4 ? 2 : m <= 8 ? 3 : m <= 16 ? 4 : 5; }

template <int FMT>
const void* kernel_of_fmt(int v) {
    switch (v) {
        case 0: return (const void*)kyb::gemv_t16_kernel<FMT, 1, 1>;
        case 1: return (const void*)kyb::gemv_t16_kernel<FMT, 1, 2>;
        case 2: return (const void*)kyb::gemv_t16_kernel<FMT, 1, 4>;
        case 3: return (const void*)kyb::gemv_t16_kernel<FMT, 1, 8>;
        case 4: return (const void*)kyb::gemv_t16_kernel<FMT, 2, 8>;
        default: return (const void*)kyb::gemv_t16_kernel<FMT, 4, 8>;
    }
}

const void* gemv_kernel_ptr(int fmt, int v) {
    switch (fmt) {
        case KYB_FMT_Q4_K: return kernel_of_fmt<KYB_FMT_Q4_K>(v);
        case KYB_FMT_Q6_K: return kernel_of_fmt<KYB_FMT_Q6_K>(v);
        case KYB_FMT_Q3_K: return kernel_of_fmt<KYB_FMT_Q3_K>(v);
        case KYB_FMT_Q5_K: return kernel_of_fmt<KYB_FMT_Q5_K>(v);
        case KYB_FMT_Q8_0: return kernel_of_fmt<KYB_FMT_Q8_0>(v);
        case KYB_FMT_Q2_K: return kernel_of_fmt<KYB_FMT_Q2_K>(v);
        case KYB_FMT_IQ4_XS: return kernel_of_fmt<KYB_FMT_IQ4_XS>(v);
        default: return kernel_of_fmt<KYB_FMT_NVFP4>(v);
    }
}

int device_sms() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        (void)cudaGetLastError();
    }
    return sms;
}

// Canonical k-chunk of a matrix: depends on (n, k) only - never on m or on the launch shape - so the partial sums of an activation row are always formed chunk by
// chunk and added in k order (bit-identical rows whatever m and however the chunks are spread over warps and CTAs). At most 8 k-blocks, so that the staged
// activations of one chunk fit in shared memory for 32 rows. Matrices with thousands of row tiles are dealt to the warps in whole row tiles and take the
// largest even division of k; smaller ones are dealt in runs of chunks and a chunk is about half of what one of ~1800 warps gets. Among the sizes near the
// target the one that divides k most evenly, then the larger.
int canonical_chunk(int ntiles, int nb) {
    const int hi = std::min(nb, 8);
    const int target = ntiles >= 3000 ? hi : std::max(1, std::min(hi, (int)((double)ntiles * nb / 3600.0 + 0.5)));
    const int from = ntiles >= 3000 ? std::max(1, hi / 2) : std::max(1, target - target / 4);
    int best = target, best_waste = 1 << 30;
    for (int kc = from; kc <= std::min(hi, target + (target + 1) / 2); ++kc) {
        const int waste = (nb + kc - 1) / kc * kc - nb;
        if (waste < best_waste || (waste == best_waste && kc > best)) best = kc, best_waste = waste;
    }
    return best;
}

// Warps per CTA, k-parts and the way work is dealt. k is split over CTAs only as far as the staged activations of a part must fit in shared memory next to the
// warps' rings. For every warp count two ways are scored by how even the busiest warp's share is: whole row tiles per warp (nothing goes through the workspace)
// or runs of chunks (chunk sums through the workspace and a finalize launch); more warps per SM are mildly preferred. Small matrices that would take the second
// way are then moved to whole row tiles per CTA with the chunk sums in shared memory (one launch), see the end of the function.
GemvPlan search_plan(int fmt, int64_t n, int64_t k, int64_t m) {
    const int sms = device_sms();
    const int nb = (int)(k / 256), ntiles = (int)((n + 15) / 16);
    const size_t smem_cap = 226 * 1024;
    const int kc = canonical_chunk(ntiles, nb), nchunks = (nb + kc - 1) / kc;
    const int v = variant_of(m), nt = VAR_NT[v], mst = VAR_MST[v];
    const int max_warps = nt <= 2 ? 12 : 8;                            // measured: 13 to 16 warps per SM are slower than 10 to 12 on every shape
    GemvPlan best{};
    double best_score = -1.0;
    for (int ksplit = 1; ksplit <= std::min(nchunks, sms); ++ksplit) {
        const int cpp = (nchunks + ksplit - 1) / ksplit;
        if ((nchunks + cpp - 1) / cpp != ksplit) continue;               // one representative per distinct split
        const int kbp = std::min(nb, cpp * kc), grid = sms / ksplit * ksplit;
        for (int warps = 4; warps <= max_warps; ++warps) {
            const size_t smem = plan_smem(fmt, nt, mst, kbp, warps, kyb::GEMV_DSTAGES);
            if (smem > smem_cap) continue;
            const double wp = (double)(grid / ksplit) * warps;                                  // warps of a part
            const double parts = (double)nchunks / ((double)ksplit * cpp);                      // the last part may be shorter
            // measured on every shape of the benchmark: 10 to 12 warps per SM are within 2 % of each other when their busiest warps carry the same load,
            // fewer than 9 or more than 12 are slower; fewer are taken only when shared memory leaves no choice (many activation rows)
            const int pref = nt <= 2 ? 10 : 6;
            const double occupancy = warps >= pref ? 1.0 : 0.45 + 0.05 * warps;
            const double common = parts * ((double)grid / sms) * occupancy * (1.0 - 0.02 * (ksplit - 1));
            for (int aligned = 0; aligned < 2; ++aligned) {
                const double upw = aligned ? ntiles / wp : (double)ntiles * cpp / wp;           // row tiles or units per warp
                const double balance = upw / std::ceil(upw);
                const double shared = aligned && ksplit == 1 ? 1.0 : 0.9;                       // cost of the workspace round trip and the finalize launch
                const double score = balance * common * shared;
                if (score > best_score) best_score = score, best = GemvPlan{nt, mst, warps, kyb::GEMV_DSTAGES, kbp, ksplit, grid, smem, kc, nchunks, cpp, aligned, 0};
            }
        }
        if (best_score > 0) break;                                        // the smallest split that fits
    }
    // Form (c) instead of form (b) where the second launch costs more than the uneven shares of whole row tiles per CTA: G = min(SMs, row tiles) CTAs own
    // floor / ceil (row tiles / G) row tiles each, so the product runs as long as its busiest CTA; against that stand about 2.5 us for the finalize launch of form (b)
    // (measured inside chained launches: 4096 x 4096 7.4 -> 5.2 us, 10240 x 5120 10.2 -> 9.1 us, 5120 x 8192 9.3 -> 8.7 us at one row; more with 8 rows).
    // The whole of k is staged in every CTA, so up to 8 activation rows and only while that fits shared memory; at least 64 CTAs must get work.
    if (best.warps > 0 && !(best.aligned && best.ksplit == 1) && ntiles >= 64 && m <= 8) {
        const int grid = std::min(sms, ntiles), rpc = (ntiles + grid - 1) / grid;
        const double t_us = (double)ntiles * nb * (double)kyb_tile_bytes(fmt) / 5.0e6;          // the product at 5 TB/s
        const double penalty_us = t_us * ((double)rpc * grid / ntiles - 1.0);
        const size_t cpart = (size_t)rpc * nchunks * (size_t)m * 16 * sizeof(float);
        if (penalty_us < 2.5) {
            for (int warps = max_warps; warps >= 8; --warps) {
                const size_t smem = plan_smem(fmt, nt, mst, nb, warps, kyb::GEMV_DSTAGES) + cpart;
                if (smem <= smem_cap) return GemvPlan{nt, mst, warps, kyb::GEMV_DSTAGES, nb, 1, grid, smem, kc, nchunks, nchunks, 0, 1};
            }
        }
    }
    return best;
}

// plans are cached per (format, n, k, m): a decode step calls this per linear
GemvPlan make_plan(int fmt, int64_t n, int64_t k, int64_t m) {
    static std::mutex mu;
    static std::map<std::tuple<int, int64_t, int64_t, int64_t>, GemvPlan> cache;
    const auto key = std::make_tuple(fmt, n, k, m);
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    const GemvPlan pl = search_plan(fmt, n, k, m);
    cache.emplace(key, pl);
    return pl;
}

// opt in to large dynamic shared memory once per device and kernel (the attribute is per device and per function)
int ensure_smem_attr(const void* kern) {
    static std::mutex mu;
    static std::unordered_map<const void*, unsigned> done;
    int dev = 0;
    KYB_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(mu);
    unsigned& mask = done[kern];
    if (!(mask & (1u << (dev & 31)))) {
        KYB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(227 * 1024 - 1024)));   // leaves room for the few static words
        mask |= 1u << (dev & 31);
    }
    return KYB_OK;
}

// launches `kern` plainly or, when chained, with programmatic stream serialization (its CTAs may become resident while the preceding kernel of the stream drains)
int launch_maybe_chained(const void* kern, dim3 grid, dim3 block, size_t smem, cudaStream_t st, void** args, bool chained, const char* what) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = chained ? 1 : 0;
    KYB_CUDA(cudaLaunchKernelExC(&cfg, kern, args));
    return kyb_launch_check(what);
}

bool two_step(const GemvPlan& pl) { return !pl.local && !(pl.aligned && pl.ksplit == 1); }     // form (b): chunk sums through the workspace, then the finalize kernel
size_t partial_bytes(const GemvPlan& pl, int64_t n, int64_t m) { return (size_t)pl.nchunks * (size_t)m * (size_t)((n + 15) / 16 * 16) * sizeof(float); }

int check_gemv_args(int fmt, const void* t16, int64_t n, int64_t k, const void* x, int64_t m, int64_t ldx) {
    KYB_REQUIRE(fmt >= 0 && fmt < KYB_FMT_COUNT, "unknown weight format %d", fmt);
    KYB_REQUIRE(n > 0 && k > 0 && k % 256 == 0, "n=%lld k=%lld: k must be a positive multiple of 256", (long long)n, (long long)k);
    KYB_REQUIRE(m >= 1 && m <= 32, "m=%lld: this entry point serves 1..32 activation rows", (long long)m);
    KYB_REQUIRE(t16 && x, "null pointer");
    KYB_REQUIRE(((uintptr_t)t16 & 15) == 0 && ((uintptr_t)x & 15) == 0, "t16 and x must be 16-byte aligned");
    KYB_REQUIRE(ldx >= k && ldx % 8 == 0, "ldx=%lld must be >= k and a multiple of 8", (long long)ldx);
    KYB_REQUIRE(n <= (int64_t)1 << 30 && k <= (int64_t)1 << 24, "matrix too large for 32-bit tile indices");
    return KYB_OK;
}

// the GEMV kernel and, in form (b), the finalize kernel behind it. partial: scratch for the chunk sums (form (b)); y == nullptr: chunk sums only
int launch_gemv(int fmt, const GemvPlan& pl, const void* t16, int64_t n, int64_t k, const void* x, int64_t m, int64_t ldx, float gscale, void* y, int64_t ldy,
                float* partial, unsigned int* status, bool chained, cudaStream_t st, const void* x2 = nullptr, float limit = 0.f) {
    const bool sums_only = y == nullptr, staged = sums_only || two_step(pl);
    kyb::GemvParams p;
    p.t16 = (const uint8_t*)t16, p.x = (const __half*)x, p.x2 = (const __half*)x2, p.limit = limit, p.y = (__half*)y, p.partial = partial, p.status = status;
    p.ldx = ldx, p.ldy = ldy, p.n = (int)n, p.npad = (int)((n + 15) / 16 * 16), p.nb = (int)(k / 256), p.m = (int)m, p.mst = pl.mst;
    p.kbp = pl.kbp, p.ksplit = pl.ksplit, p.warps = pl.warps, p.stages = pl.stages, p.gscale = gscale, p.kc = pl.kc, p.nchunks = pl.nchunks, p.cpp = pl.cpp, p.aligned = pl.aligned;
    p.partial_only = (staged || pl.local) ? 1 : 0, p.pdl = chained ? 1 : 0;
    p.local = (pl.local && !sums_only) ? 1 : 0;                    // chunk sums asked for by the caller go to its buffer as in form (b)
    const void* kern = gemv_kernel_ptr(fmt, variant_of(m));
    if (int rc = ensure_smem_attr(kern)) return rc;
    void* args[] = {(void*)&p};
    if (int rc = launch_maybe_chained(kern, dim3((unsigned)pl.grid), dim3((unsigned)pl.warps * 32), pl.smem, st, args, chained, "gemv_t16")) return rc;
    if (staged && !sums_only) {
        const int64_t tot = m * n;
        const float* part = partial;
        int nchunks = pl.nchunks, mi = (int)m, ni = (int)n, npad_i = p.npad;
        __half* yp = (__half*)y;
        void* fargs[] = {(void*)&part, (void*)&nchunks, (void*)&mi, (void*)&ni, (void*)&npad_i, (void*)&gscale, (void*)&yp, (void*)&ldy};
        return launch_maybe_chained((const void*)kyb::gemv_finalize_kernel, dim3((unsigned)((tot + 255) / 256)), dim3(256), 0, st, fargs, chained, "gemv_finalize");
    }
    return KYB_OK;
}

}  // namespace

extern "C" int kyb_gemv_plan(int fmt, int64_t n, int64_t k, int64_t m, int* out8) {
    KYB_REQUIRE(fmt >= 0 && fmt < KYB_FMT_COUNT && n > 0 && k > 0 && k % 256 == 0 && m >= 1 && m <= 32 && out8, "bad arguments");
    const GemvPlan pl = make_plan(fmt, n, k, m);
    out8[0] = pl.nt, out8[1] = pl.local ? 2 : pl.aligned, out8[2] = pl.warps, out8[3] = pl.kc, out8[4] = pl.kbp, out8[5] = pl.ksplit, out8[6] = (int)pl.smem, out8[7] = pl.grid;
    return KYB_OK;
}

extern "C" size_t kyb_gemv_workspace_bytes(int fmt, int64_t n, int64_t k, int64_t m) {
    if (fmt < 0 || fmt >= KYB_FMT_COUNT || n <= 0 || k <= 0 || k % 256 || m <= 0 || m > 32) return 0;
    const GemvPlan pl = make_plan(fmt, n, k, m);
    return two_step(pl) ? partial_bytes(pl, n, m) : 0;
}

extern "C" int kyb_gemv_t16(int fmt, const void* t16, int64_t n, int64_t k, const void* x, int64_t m, int64_t ldx, float gscale, void* y, int64_t ldy,
                            void* workspace, size_t workspace_bytes, int flags, void* stream) {
    if (int rc = check_gemv_args(fmt, t16, n, k, x, m, ldx)) return rc;
    KYB_REQUIRE(y && ldy >= n, "y is null or ldy=%lld < n", (long long)ldy);
    KYB_REQUIRE((flags & ~KYB_GEMV_CHAINED) == 0, "unknown flags 0x%x", flags);
    const GemvPlan pl = make_plan(fmt, n, k, m);
    KYB_REQUIRE(pl.warps > 0, "no launch configuration fits shared memory for k=%lld m=%lld", (long long)k, (long long)m);
    const size_t need = two_step(pl) ? partial_bytes(pl, n, m) : 0;
    if (need && (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 15))) {
        kyb_set_error("gemv needs %zu bytes of 16-byte aligned workspace, got %zu", need, workspace ? workspace_bytes : (size_t)0);
        return KYB_EWORKSPACE;
    }
    unsigned int* status = kyb_device_status_word();
    KYB_REQUIRE(status, "could not set up the device status word");
    return launch_gemv(fmt, pl, t16, n, k, x, m, ldx, gscale, y, ldy, (float*)workspace, status, (flags & KYB_GEMV_CHAINED) != 0, (cudaStream_t)stream);
}

// The same product on a gated input: row r fed to the product is fp16(silu(a[r]) * b[r]) (fp32 arithmetic, saturated, optional clamp), formed while the rows are
// staged, so the activation kernel and its round trip through HBM disappear. Replaces kyojin_mlx/foreign_linear.py:960-977 `DevPack.apply_glu`.
extern "C" int kyb_gemv_glu_t16(int fmt, const void* t16, int64_t n, int64_t k, const void* a, const void* b, float limit, int64_t m, int64_t ldx, float gscale, void* y,
                                int64_t ldy, void* workspace, size_t workspace_bytes, int flags, void* stream) {
    if (int rc = check_gemv_args(fmt, t16, n, k, a, m, ldx)) return rc;
    KYB_REQUIRE(b && ((uintptr_t)b & 15) == 0, "b is null or not 16-byte aligned");
    KYB_REQUIRE(y && ldy >= n, "y is null or ldy=%lld < n", (long long)ldy);
    KYB_REQUIRE((flags & ~KYB_GEMV_CHAINED) == 0, "unknown flags 0x%x", flags);
    const GemvPlan pl = make_plan(fmt, n, k, m);
    KYB_REQUIRE(pl.warps > 0, "no launch configuration fits shared memory for k=%lld m=%lld", (long long)k, (long long)m);
    const size_t need = two_step(pl) ? partial_bytes(pl, n, m) : 0;
    if (need && (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 15))) {
        kyb_set_error("gemv needs %zu bytes of 16-byte aligned workspace, got %zu", need, workspace ? workspace_bytes : (size_t)0);
        return KYB_EWORKSPACE;
    }
    unsigned int* status = kyb_device_status_word();
    KYB_REQUIRE(status, "could not set up the device status word");
    return launch_gemv(fmt, pl, t16, n, k, a, m, ldx, gscale, y, ldy, (float*)workspace, status, (flags & KYB_GEMV_CHAINED) != 0, (cudaStream_t)stream, b, limit);
}

// Two-step form with the partial sums exposed (chunk sums, then finalize): the call shape of the reference's few-row MMA GEMV,
// kyojin_mlx/mma_gemv.py:129-149 `partial_mma` -> f32 [parts, rows, n] and `finalize_rows` -> [rows, n]. partial: f32 [kyb_gemv_chunks(n, k)][m][npad].
extern "C" int kyb_gemv_chunks(int64_t n, int64_t k) {
    if (n <= 0 || k <= 0 || k % 256) return 0;
    const int nb = (int)(k / 256), kc = canonical_chunk((int)((n + 15) / 16), nb);
    return (nb + kc - 1) / kc;
}

extern "C" int kyb_gemv_partial_t16(int fmt, const void* t16, int64_t n, int64_t k, const void* x, int64_t m, int64_t ldx, void* partial, void* stream) {
    if (int rc = check_gemv_args(fmt, t16, n, k, x, m, ldx)) return rc;
    KYB_REQUIRE(partial, "null pointer");
    const GemvPlan pl = make_plan(fmt, n, k, m);
    KYB_REQUIRE(pl.warps > 0, "no launch configuration fits shared memory for k=%lld m=%lld", (long long)k, (long long)m);
    unsigned int* status = kyb_device_status_word();
    KYB_REQUIRE(status, "could not set up the device status word");
    return launch_gemv(fmt, pl, t16, n, k, x, m, ldx, 1.0f, nullptr, 0, (float*)partial, status, false, (cudaStream_t)stream);
}

extern "C" int kyb_gemv_finalize(const void* partial, int chunks, int64_t m, int64_t n, float gscale, void* y, int64_t ldy, void* stream) {
    KYB_REQUIRE(partial && y && chunks > 0 && m > 0 && n > 0 && ldy >= n, "bad arguments");
    const int64_t tot = m * n;
    kyb::gemv_finalize_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const float*)partial, chunks, (int)m, (int)n, (int)((n + 15) / 16 * 16), gscale,
                                                                                              (__half*)y, ldy);
    return kyb_launch_check("gemv_finalize");
}

// ------------------------------------------------------------------------------------------------ decode GEMV without any allocation
// Some hosts may not allocate device memory at the moment they need a GEMV: a serving process that handed every free byte of HBM to its KV-cache
// pool at start-up (a later cudaMalloc fails or fragments the pool), a latency-critical decode loop that cannot take the implicit device
// synchronisation of cudaMalloc / cudaFree, or an embedding runtime whose plug-in contract forbids the callee to allocate. For them the scratch of
// this variant (chunk sums, timeout word) lives in a fixed array that is part of the library image: every GPU that loads the library holds
// KYB_GEMV_STATIC_SCRATCH_BYTES + 256 bytes of it until the process exits.
#define KYB_GEMV_STATIC_SCRATCH_BYTES (16u << 20)
// [0, 256): status word (zero when the library is loaded; a successful call never writes it); then the fp32 chunk sums
static __device__ __align__(256) unsigned char g_gemv_static_scratch[256 + KYB_GEMV_STATIC_SCRATCH_BYTES];

namespace {
// In host code the array's name is only a stand-in; the device address is looked up once per device (with that device current) and cached.
int static_scratch_address(unsigned char** out) {
    static std::mutex mu;
    static unsigned char* addr[64] = {nullptr};
    int dev = 0;
    KYB_CUDA(cudaGetDevice(&dev));
    KYB_REQUIRE(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lk(mu);
    if (!addr[dev]) {
        void* ptr = nullptr;
        KYB_CUDA(cudaGetSymbolAddress(&ptr, g_gemv_static_scratch));
        addr[dev] = (unsigned char*)ptr;
    }
    *out = addr[dev];
    return KYB_OK;
}
}  // namespace

extern "C" int kyb_gemv_t16_static(int fmt, const void* t16, int64_t n, int64_t k, const void* x, int64_t m, int64_t ldx, float gscale, void* y, int64_t ldy,
                                   int check, void* stream) {
    if (int rc = check_gemv_args(fmt, t16, n, k, x, m, ldx)) return rc;
    KYB_REQUIRE(y && ldy >= n, "y is null or ldy=%lld < n", (long long)ldy);
    const GemvPlan pl = make_plan(fmt, n, k, m);
    KYB_REQUIRE(pl.warps > 0, "no launch configuration fits shared memory for k=%lld m=%lld", (long long)k, (long long)m);
    const size_t need = two_step(pl) ? partial_bytes(pl, n, m) : 0;
    if (need > KYB_GEMV_STATIC_SCRATCH_BYTES) {
        kyb_set_error("kyb_gemv_t16_static: this shape needs %zu bytes of chunk sums, the built-in array holds %u; use kyb_gemv_t16 with a caller workspace", need,
                      (unsigned)KYB_GEMV_STATIC_SCRATCH_BYTES);
        return KYB_EWORKSPACE;
    }
    unsigned char* base = nullptr;
    if (int rc = static_scratch_address(&base)) return rc;
    unsigned int* status = (unsigned int*)base;
    float* partial = (float*)(base + 256);
    cudaStream_t st = (cudaStream_t)stream;
    // every chunk sum the finalize pass reads was written by the launch before it, so nothing in the array has to start at zero
    if (int rc = launch_gemv(fmt, pl, t16, n, k, x, m, ldx, gscale, y, ldy, partial, status, false, st)) return rc;
    if (check) {
        unsigned int v = 0;
        KYB_CUDA(cudaMemcpyAsync(&v, status, sizeof(v), cudaMemcpyDeviceToHost, st));
        KYB_CUDA(cudaStreamSynchronize(st));
        if (v) {
            KYB_CUDA(cudaMemsetAsync(status, 0, sizeof(v), st));                // the word must read zero again for the next call
            kyb_set_error("device status 0x%x: a kernel gave up a bounded wait", v);
            return KYB_ETIMEOUT;
        }
    }
    return KYB_OK;
}

// ------------------------------------------------------------------------------------------------ routed experts (host side)
extern "C" int kyb_moe_groups(const void* eids, int64_t S, int E, void* g_expert, void* g_slots, void* ngroups, void* stream) {
    KYB_REQUIRE(eids && g_expert && g_slots && ngroups, "null pointer");
    KYB_REQUIRE(S > 0 && S <= (1 << 20) && E > 0 && E <= 8192, "S=%lld E=%d out of range", (long long)S, E);
    kyb::moe_groups_kernel<<<1, 1024, (size_t)(2 * E + 1) * sizeof(uint32_t), (cudaStream_t)stream>>>((const uint32_t*)eids, (int)S, E, (uint32_t*)g_expert, (uint32_t*)g_slots,
                                                                                                    (uint32_t*)ngroups);
    return kyb_launch_check("moe_groups");
}

extern "C" int kyb_gemv_group_t16(int fmt, const void* t16, const void* t16b, int64_t n, int64_t k, int E, const void* x, const void* x2, float limit, int64_t ldx,
                                  const void* eids, const void* xrows, int xdiv, int64_t S, const void* gs, const void* gsb, void* y, int64_t ldy, const void* g_expert,
                                  const void* g_slots, const void* ngroups, void* stream) {
    KYB_REQUIRE(fmt >= 0 && fmt < KYB_FMT_COUNT, "unknown weight format %d", fmt);
    KYB_REQUIRE(n > 0 && n % 16 == 0 && k > 0 && k % 256 == 0 && E > 0, "n=%lld k=%lld: expert matrices need n %% 16 == 0 and k %% 256 == 0", (long long)n, (long long)k);
    KYB_REQUIRE(t16 && x && y && g_expert && g_slots && ngroups, "null pointer");
    KYB_REQUIRE(S > 0 && S < (1ll << 30) && xdiv > 0 && ldx >= k && ldx % 8 == 0 && ldy >= n, "S=%lld xdiv=%d ldx=%lld ldy=%lld", (long long)S, xdiv, (long long)ldx, (long long)ldy);
    KYB_REQUIRE(((uintptr_t)t16 & 15) == 0 && ((uintptr_t)t16b & 15) == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)x2 & 15) == 0, "t16, x (and t16b, x2) must be 16-byte aligned");
    unsigned int* status = kyb_device_status_word();
    KYB_REQUIRE(status, "could not set up the device status word");
    const int nb = (int)(k / 256), ntiles = (int)(n / 16), sms = device_sms();
    int warps = 0;
    size_t smem = 0;
    for (int w = 16; w >= 4; w -= 4) {
        smem = plan_smem(fmt, 1, 8, nb, w, kyb::GEMV_STAGES);
        if (smem <= 226 * 1024 - 256) {
            warps = w;
            break;
        }
    }
    KYB_REQUIRE(warps > 0, "k=%lld: the staged activations of a group do not fit in shared memory", (long long)k);
    warps = std::min(warps, std::max(4, (ntiles + 3) / 4 * 4));
    const int64_t exp_groups = std::max<int64_t>(1, std::min<int64_t>(S, E)) * (t16b ? 2 : 1);
    int rc = (int)std::min<int64_t>(std::max<int64_t>(1, (4 * sms + exp_groups - 1) / exp_groups), std::max(1, ntiles / warps));
    kyb::GroupParams p;
    p.t16 = (const uint8_t*)t16, p.t16b = (const uint8_t*)t16b, p.x = (const __half*)x, p.x2 = (const __half*)x2, p.eids = (const uint32_t*)eids, p.xrows = (const uint32_t*)xrows;
    p.g_expert = (const uint32_t*)g_expert, p.g_slots = (const uint32_t*)g_slots;
    p.ngroups = (const uint32_t*)ngroups, p.gs = (const float*)gs, p.gsb = (const float*)gsb, p.y = (__half*)y, p.status = status, p.ldx = ldx, p.ldy = ldy, p.limit = limit;
    p.n = (int)n, p.nb = nb, p.kc = canonical_chunk(ntiles, nb), p.xdiv = xdiv, p.rc = rc, p.warps = warps, p.S = (int)S, p.E = E;
    const void* kern = fmt == KYB_FMT_Q4_K   ? (const void*)kyb::gemv_group_kernel<KYB_FMT_Q4_K>
                       : fmt == KYB_FMT_Q6_K ? (const void*)kyb::gemv_group_kernel<KYB_FMT_Q6_K>
                       : fmt == KYB_FMT_Q3_K ? (const void*)kyb::gemv_group_kernel<KYB_FMT_Q3_K>
                       : fmt == KYB_FMT_Q5_K ? (const void*)kyb::gemv_group_kernel<KYB_FMT_Q5_K>
                       : fmt == KYB_FMT_Q8_0 ? (const void*)kyb::gemv_group_kernel<KYB_FMT_Q8_0>
                       : fmt == KYB_FMT_Q2_K ? (const void*)kyb::gemv_group_kernel<KYB_FMT_Q2_K>
                       : fmt == KYB_FMT_IQ4_XS ? (const void*)kyb::gemv_group_kernel<KYB_FMT_IQ4_XS>
                                             : (const void*)kyb::gemv_group_kernel<KYB_FMT_NVFP4>;
    if (int r = ensure_smem_attr(kern)) return r;
    void* args[] = {(void*)&p};
    KYB_CUDA(cudaLaunchKernel(kern, dim3((unsigned)sms), dim3((unsigned)warps * 32), args, smem + 64, (cudaStream_t)stream));
    return KYB_OK;
}
