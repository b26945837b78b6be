// Routed-expert plumbing around the quantized products: router softmax / top-k, slot sort by expert (counting sort), row gather, gated
// activation, weighted combine. These are launch-bound elementwise / index kernels; the arithmetic follows the reference's Metal kernels
// (kyojin_mlx/foreign_moe.py:77-119 _SELECT / _SILU / _COMBINE, foreign_kqgmm.py:169-188 _CSORT, :242-261 _GATHER_ORD / _SILU_PERM,
// moe_sort.py:18-45) in float32.
#include <cooperative_groups.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdlib>

#include "kyb_common.cuh"

namespace kyb {

// One warp per token. logits fp32 [T, ld]: E expert logits, then (has_shared) the shared-expert gate logit at column E.
// softmax in fp32 (exp(l - max) * (1 / sum)), k rounds of arg-max by value, lowest index on ties, weights top / sum(top) when norm.
__global__ void moe_select_kernel(const float* __restrict__ lg, int64_t ld, int T, int E, int K, int norm, int has_shared, uint32_t* __restrict__ inds,
                                  float* __restrict__ scs, float* __restrict__ sgs) {
    extern __shared__ float sp[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    const int t = blockIdx.x * wpb + warp;
    if (t >= T) return;
    float* p = sp + (size_t)warp * E;
    const float* L = lg + (size_t)t * ld;
    float m = -INFINITY;
    for (int i = lane; i < E; i += 32) {
        const float v = L[i];
        p[i] = v;
        m = fmaxf(m, v);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float sum = 0.f;
    for (int i = lane; i < E; i += 32) {
        const float e = expf(p[i] - m);
        p[i] = e;
        sum += e;
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.0f / sum;
    for (int i = lane; i < E; i += 32) p[i] *= inv;
    __syncwarp();
    float ts = 0.f, mine = 0.f;                      // lane k keeps the k-th weight (K <= 32)
    for (int k = 0; k < K; ++k) {
        float best = -1.0f;
        uint32_t bi = 0xFFFFFFFFu;
        for (int i = lane; i < E; i += 32)
            if (p[i] > best) best = p[i], bi = (uint32_t)i;
        float gv = best;
#pragma unroll
        for (int o = 16; o; o >>= 1) gv = fmaxf(gv, __shfl_xor_sync(0xffffffffu, gv, o));
        uint32_t gi = best == gv ? bi : 0xFFFFFFFFu;
#pragma unroll
        for (int o = 16; o; o >>= 1) gi = min(gi, __shfl_xor_sync(0xffffffffu, gi, o));
        if (gi < (uint32_t)E && (gi & 31u) == (uint32_t)lane) p[gi] = -1.0f;
        __syncwarp();
        ts += gv;
        if (lane == k) mine = gv;
        if (lane == 0) inds[(size_t)t * K + k] = gi;
    }
    if (lane < K) scs[(size_t)t * K + lane] = norm ? mine / ts : mine;
    if (lane == 0 && sgs) sgs[t] = has_shared ? 1.0f / (1.0f + expf(-L[E])) : 0.0f;
}

// Counting sort of P slots by expert by ONE thread-block cluster (1 CTA for a few thousand slots, 8 CTAs beyond): every CTA takes a contiguous share of
// the slots and counts them per expert in its shared memory; after a cluster barrier every CTA reads all the CTAs' counts through distributed shared memory,
// forms the segment starts with a parallel scan over the experts (no serial pass, no scratch in global memory) and the start of its own share inside every
// segment; then it scatters its slots with shared-memory cursors. rank (optional) maps expert -> position of its segment.
// Outputs (any may be null): order[pos] = slot, inv[slot] = pos, tok[pos] = slot / topk, ids_s[pos] = expert, wts_s[pos] = wts[slot],
// off[E + 1] = first row of each segment, tb[E + 1] = first tile of each segment for tiles of mt rows.
// Slots whose id is outside [0, E) (the router writes 0xFFFFFFFF for a token with NaN logits) belong to no segment: they take the positions
// [off[E], P) behind the last segment, with weight 0, so that order / inv stay permutations and every output entry is written.
constexpr int PLAN_THREADS = 1024, PLAN_PER = 9;                     // experts per thread in the scan: E + 1 <= 1024 * 9

// exclusive scan of one value per thread over the CTA (1024 threads); `carry` = a shared array of 33 words
__device__ __forceinline__ uint32_t block_excl_scan(uint32_t v, uint32_t* carry, uint32_t& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    if (lane == 31) carry[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        uint32_t w = carry[lane], wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t n = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += n;
        }
        carry[lane] = wi - w;
        if (lane == 31) carry[32] = wi;
    }
    __syncthreads();
    total = carry[32];
    const uint32_t out = carry[warp] + inc - v;
    __syncthreads();                                                  // carry is reused by the next scan
    return out;
}

__global__ void __launch_bounds__(PLAN_THREADS) moe_plan_kernel(const int32_t* __restrict__ ids, const float* __restrict__ wts, const uint32_t* __restrict__ rank, int E, int P,
                                                                int topk, int mt, uint32_t* __restrict__ order, uint32_t* __restrict__ inv, uint32_t* __restrict__ tok,
                                                                int32_t* __restrict__ ids_s, float* __restrict__ wts_s, uint32_t* __restrict__ off, uint32_t* __restrict__ tb) {
    namespace cg = cooperative_groups;
    extern __shared__ uint32_t sm[];
    uint32_t* counts = sm;             // [E + 1]: this CTA's slots per segment; entry E = slots that belong to no expert
    uint32_t* cursor = sm + E + 1;     // [E + 1]: where this CTA's next slot of a segment goes
    uint32_t* carry = cursor + E + 1;  // [33]
    cg::cluster_group cl = cg::this_cluster();
    const int R = (int)cl.num_blocks(), r = (int)cl.block_rank();
    const int share = (P + R - 1) / R, p0 = min(P, r * share), p1 = min(P, p0 + share);
    auto key_of = [&](int e) -> uint32_t { return (e >= 0 && e < E) ? (rank ? rank[e] : (uint32_t)e) : (uint32_t)E; };
    for (int e = threadIdx.x; e <= E; e += blockDim.x) counts[e] = 0u;
    __syncthreads();
    for (int p = p0 + threadIdx.x; p < p1; p += blockDim.x) atomicAdd(&counts[key_of(ids[p])], 1u);
    cl.sync();                                                        // every CTA's counts are complete and visible to the cluster
    // thread t owns segments [t * PLAN_PER, (t + 1) * PLAN_PER): their sizes over all CTAs and what the CTAs before this one put into them
    uint32_t tot[PLAN_PER], bef[PLAN_PER], rows = 0, tiles = 0;
#pragma unroll
    for (int j = 0; j < PLAN_PER; ++j) {
        const int e = threadIdx.x * PLAN_PER + j;
        tot[j] = bef[j] = 0u;
        if (e <= E)
            for (int c = 0; c < R; ++c) {
                const uint32_t v = cl.map_shared_rank(counts, c)[e];
                tot[j] += v;
                if (c < r) bef[j] += v;
            }
        rows += tot[j];
        if (e < E) tiles += (tot[j] + (uint32_t)mt - 1u) / (uint32_t)mt;
    }
    uint32_t all_rows, all_tiles;
    uint32_t row0 = block_excl_scan(rows, carry, all_rows), tile0 = block_excl_scan(tiles, carry, all_tiles);
#pragma unroll
    for (int j = 0; j < PLAN_PER; ++j) {
        const int e = threadIdx.x * PLAN_PER + j;
        if (e <= E) {
            cursor[e] = row0 + bef[j];
            if (r == 0) {
                if (off) off[e] = row0;
                if (tb) tb[e] = tile0;
            }
            row0 += tot[j];
            if (e < E) tile0 += (tot[j] + (uint32_t)mt - 1u) / (uint32_t)mt;
        }
    }
    cl.sync();                                                        // nobody reads a peer's counts after this point (a CTA may leave while others scatter)
    for (int p = p0 + threadIdx.x; p < p1; p += blockDim.x) {
        const int e0 = ids[p];
        const bool valid = e0 >= 0 && e0 < E;
        const uint32_t pos = atomicAdd(&cursor[key_of(e0)], 1u);
        if (order) order[pos] = (uint32_t)p;
        if (inv) inv[p] = pos;
        if (tok) tok[pos] = (uint32_t)(p / topk);
        if (ids_s) ids_s[pos] = e0;
        if (wts_s && wts) wts_s[pos] = valid ? wts[p] : 0.0f;
    }
}

// ---- router logits on the tensor cores. An fp32 gate row w is cut into three fp16 pieces of s w (s = a power of two per row that puts the row's largest
// magnitude in [2^13, 2^14)): s w = hi + 2^-11 mid + 2^-22 lo with hi = fp16(s w), mid = fp16(2^11 (s w - hi)), lo = fp16(2^11 (2^11 (s w - hi) - mid)); every
// difference is exact in fp32, so the three pieces carry the 24 bits of w (entries more than 2^27 below the row's maximum lose low bits; they do not matter to
// a logit). With fp16 activations every product piece * x is exact in the fp32 accumulator of the MMA, and
//     logit = (x . hi + 2^-11 x . mid + 2^-22 x . lo) / s.
// pieces: fp16 [3 * rpad, H], piece p of row r at row p * rpad + r; rows [R, rpad) are zero. inv_scale[r] = 1 / s.
__global__ void router_split_kernel(const float* __restrict__ gw, const float* __restrict__ sgw, int E, int R, int rpad, int H, __half* __restrict__ pieces,
                                    float* __restrict__ inv_scale) {
    const int r = blockIdx.x;
    __shared__ float red[32];
    const float* w = r < E ? gw + (size_t)r * H : (r < R ? sgw : nullptr);
    float mx = 0.f;
    if (w)
        for (int c = threadIdx.x; c < H; c += blockDim.x) mx = fmaxf(mx, fabsf(w[c]));
    for (int d = 16; d; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) mx = fmaxf(mx, red[i]);
    int e = 0;
    if (mx > 0.f && mx < 3.0e38f) (void)frexpf(mx, &e);                       // mx = f 2^e, 0.5 <= f < 1: s = 2^(14 - e) puts s mx in [2^13, 2^14)
    const float sc = ldexpf(1.0f, 14 - e);
    if (threadIdx.x == 0) inv_scale[r] = ldexpf(1.0f, e - 14);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = w ? w[c] * sc : 0.f;
        const __half hi = __float2half_rn(v);
        const float r1 = (v - __half2float(hi)) * 2048.0f;
        const __half mid = __float2half_rn(r1);
        const __half lo = __float2half_rn((r1 - __half2float(mid)) * 2048.0f);
        pieces[(size_t)r * H + c] = hi;
        pieces[((size_t)rpad + r) * H + c] = mid;
        pieces[((size_t)2 * rpad + r) * H + c] = lo;
    }
}

// lg[t, c] = (d[t, c] + 2^-11 d[t, rpad + c] + 2^-22 d[t, 2 rpad + c]) * inv_scale[c]: the three partial products of the pieces, smallest first
__global__ void router_combine_kernel(const float* __restrict__ d, int64_t ldd, const float* __restrict__ inv_scale, int T, int R, int rpad, float* __restrict__ lg,
                                      int64_t ldl) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)T * R) return;
    const int t = (int)(i / R), c = (int)(i % R);
    const float* row = d + (size_t)t * ldd;
    lg[(size_t)t * ldl + c] = ((row[2 * rpad + c] * (1.0f / 2048.0f) + row[rpad + c]) * (1.0f / 2048.0f) + row[c]) * inv_scale[c];
}

// out[r, :] = x[src[r] / div, perm ? perm[c] : c]   (fp16 rows of k columns; 8 columns per thread). A source row outside [0, xrows) gives a row of zeros.
__global__ void gather_rows_kernel(const __half* __restrict__ x, int64_t ldx, int64_t xrows, const uint32_t* __restrict__ src, int div, const uint32_t* __restrict__ perm, int R,
                                   int k, __half* __restrict__ out, int64_t ldo) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int kv = k >> 3;
    if (i >= (int64_t)R * kv) return;
    const int r = (int)(i / kv), c = (int)(i % kv) * 8;
    const uint32_t srow = src[r] / (uint32_t)div;
    if ((int64_t)srow >= xrows) {
        *reinterpret_cast<uint4*>(out + (size_t)r * ldo + c) = make_uint4(0u, 0u, 0u, 0u);
        return;
    }
    const __half* xr = x + (size_t)srow * ldx;
    if (!perm) {
        *reinterpret_cast<uint4*>(out + (size_t)r * ldo + c) = *reinterpret_cast<const uint4*>(xr + c);
    } else {
        __half v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = xr[perm[c + j]];
        *reinterpret_cast<uint4*>(out + (size_t)r * ldo + c) = *reinterpret_cast<uint4*>(v);
    }
}

// h = fp16(silu(a) * b) in fp32, silu(a) = a * (1 / (1 + exp(-a))); limit > 0: a = min(a, limit), b = clamp(b, -limit, limit)
// (kyojin_mlx/foreign_linear.py:1353-1361 `_glu`, foreign_metal.py:1107-1113). Optional column permutation of the output.
__global__ void silu_mul_kernel(const __half* __restrict__ a, const __half* __restrict__ b, int64_t ld, int64_t total, int n, float limit, const uint32_t* __restrict__ perm,
                                __half* __restrict__ h, int64_t ldh) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int64_t r = i / n;
    const int c = (int)(i % n), cs = perm ? (int)perm[c] : c;
    float av = __half2float(a[r * ld + cs]), bv = __half2float(b[r * ld + cs]);
    if (limit > 0.f) av = fminf(av, limit), bv = fminf(fmaxf(bv, -limit), limit);
    h[r * ldh + c] = sat_half(av * (1.0f / (1.0f + expf(-av))) * bv);
}

// the same on 8 consecutive columns per thread (16-byte loads and stores): n, ld, ldh multiples of 8, 16-byte aligned bases, no permutation
__global__ void silu_mul8_kernel(const __half* __restrict__ a, const __half* __restrict__ b, int64_t ld, int64_t total8, int n8, float limit, __half* __restrict__ h, int64_t ldh) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total8) return;
    const int64_t r = i / n8;
    const int c = (int)(i % n8) * 8;
    const uint4 av4 = __ldg(reinterpret_cast<const uint4*>(a + r * ld + c)), bv4 = __ldg(reinterpret_cast<const uint4*>(b + r * ld + c));
    const __half* ah = reinterpret_cast<const __half*>(&av4);
    const __half* bh = reinterpret_cast<const __half*>(&bv4);
    __half o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float av = __half2float(ah[j]), bv = __half2float(bh[j]);
        if (limit > 0.f) av = fminf(av, limit), bv = fminf(fmaxf(bv, -limit), limit);
        o[j] = sat_half(av * (1.0f / (1.0f + expf(-av))) * bv);
    }
    *reinterpret_cast<uint4*>(h + r * ldh + c) = *reinterpret_cast<const uint4*>(o);
}

// o[t, c] = sum_k f32(y[t K + k, c]) * scs[t K + k] (+ sgs[t] * shared[t, c]); fp16 saturated or fp32 output (foreign_moe.py:112-119)
template <typename OUT>
__global__ void moe_combine_kernel(const __half* __restrict__ y, int64_t ldy, const float* __restrict__ scs, const float* __restrict__ sgs, const __half* __restrict__ shared,
                                   int64_t lds, int T, int K, int H, OUT* __restrict__ o, int64_t ldo) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)T * H) return;
    const int t = (int)(i / H), c = (int)(i % H);
    float acc = 0.f;
    for (int k = 0; k < K; ++k) acc += __half2float(y[((size_t)t * K + k) * ldy + c]) * scs[(size_t)t * K + k];
    if (shared) acc += sgs[t] * __half2float(shared[(size_t)t * lds + c]);
    if constexpr (sizeof(OUT) == 2) o[(size_t)t * ldo + c] = sat_half(acc);
    else o[(size_t)t * ldo + c] = acc;
}

// Router logits in fp32: lg[t, r] = sum_h gw[r, h] * float(x[t, h]) for r < E, and the shared-expert gate row sgw at r = E (kyojin_mlx/foreign_moe.py:36-75).
// A CTA keeps TT token rows in shared memory in their own type and every warp walks weight rows, so a weight row read from L2 serves TT tokens.
template <typename XT> struct XVec4;
template <> struct XVec4<float> {
    using Raw = float4;
    static __device__ __forceinline__ Raw ldraw(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
    static __device__ __forceinline__ float4 cvt(Raw v) { return v; }
    static __device__ __forceinline__ float4 ld(const float* p) { return *reinterpret_cast<const float4*>(p); }
};
template <> struct XVec4<__half> {
    using Raw = uint2;
    static __device__ __forceinline__ Raw ldraw(const __half* p) { return __ldg(reinterpret_cast<const uint2*>(p)); }
    static __device__ __forceinline__ float4 cvt(Raw v) {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ float4 ld(const __half* p) { return cvt(*reinterpret_cast<const uint2*>(p)); }
};
template <> struct XVec4<__nv_bfloat16> {
    using Raw = uint2;
    static __device__ __forceinline__ Raw ldraw(const __nv_bfloat16* p) { return __ldg(reinterpret_cast<const uint2*>(p)); }
    static __device__ __forceinline__ float4 cvt(Raw v) {
        return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u));
    }
    static __device__ __forceinline__ float4 ld(const __nv_bfloat16* p) { return cvt(*reinterpret_cast<const uint2*>(p)); }
};

// the combine on 8 consecutive columns per thread: the same sum in the same order (k ascending, then the shared expert), 16-byte loads
template <typename OUT>
__global__ void moe_combine8_kernel(const __half* __restrict__ y, int64_t ldy, const float* __restrict__ scs, const float* __restrict__ sgs, const __half* __restrict__ shared,
                                    int64_t lds, int T, int K, int H8, OUT* __restrict__ o, int64_t ldo) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)T * H8) return;
    const int t = (int)(i / H8), c = (int)(i % H8) * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k = 0; k < K; ++k) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(y + ((size_t)t * K + k) * ldy + c));
        const __half* vh = reinterpret_cast<const __half*>(&v);
        const float w = scs[(size_t)t * K + k];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += __half2float(vh[j]) * w;
    }
    if (shared) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(shared + (size_t)t * lds + c));
        const __half* vh = reinterpret_cast<const __half*>(&v);
        const float w = sgs[t];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += w * __half2float(vh[j]);
    }
    if constexpr (sizeof(OUT) == 2) {
        __half oh[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) oh[j] = sat_half(acc[j]);
        *reinterpret_cast<uint4*>(o + (size_t)t * ldo + c) = *reinterpret_cast<const uint4*>(oh);
    } else {
        float4* op = reinterpret_cast<float4*>(o + (size_t)t * ldo + c);
        op[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        op[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
}

// two fp32 multiply-adds in one instruction (sm_100: fma.rn.f32x2 on register pairs)
__device__ __forceinline__ unsigned long long ffma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long p;
    asm("mov.b64 %0, {%1, %2};" : "=l"(p) : "f"(lo), "f"(hi));
    return p;
}
__device__ __forceinline__ float sum2(unsigned long long p) {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p));
    return lo + hi;
}

template <typename XT, int TT>
__global__ void __launch_bounds__(512) router_logits_kernel(const XT* __restrict__ x, int64_t ldx, const float* __restrict__ gw, const float* __restrict__ sgw, int T, int E, int H,
                                                            float* __restrict__ lg, int64_t ldl) {
    extern __shared__ __align__(16) unsigned char router_smem[];
    XT* xs = reinterpret_cast<XT*>(router_smem);
    constexpr int PER = 16 / (int)sizeof(XT);                              // elements per 16-byte copy
    constexpr int RE = 4;                                                  // weight rows per warp pass: a token chunk read from shared memory serves 4 rows
    const int t0 = blockIdx.x * TT;
    for (int idx = threadIdx.x; idx < TT * (H / PER); idx += blockDim.x) {
        const int j = idx / (H / PER), c = idx - j * (H / PER);
        const int t = min(t0 + j, T - 1);                                   // rows past T repeat the last token; their results are not stored
        *reinterpret_cast<uint4*>(xs + (size_t)j * H + (size_t)c * PER) = *reinterpret_cast<const uint4*>(x + (size_t)t * ldx + (size_t)c * PER);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, R = E + (sgw ? 1 : 0), nw = blockDim.x >> 5;
    // weight rows are dealt to (blockIdx.y, warp) in groups of RE
    for (int r0 = (blockIdx.y * nw + warp) * RE; r0 < R; r0 += gridDim.y * nw * RE) {
        const float4* wp[RE];
#pragma unroll
        for (int e = 0; e < RE; ++e) {
            const int r = min(r0 + e, R - 1);                               // a short last group repeats its last row; the repeats are not stored
            wp[e] = reinterpret_cast<const float4*>(r < E ? gw + (size_t)r * H : sgw);
        }
        // every accumulator is a pair (sum over even inputs, sum over odd inputs) so that one packed instruction does two multiply-adds
        unsigned long long acc[RE][TT];
#pragma unroll
        for (int e = 0; e < RE; ++e)
#pragma unroll
            for (int j = 0; j < TT; ++j) acc[e][j] = 0ull;
        for (int i = lane; i < H / 4; i += 32) {
            unsigned long long wlo[RE], whi[RE];
#pragma unroll
            for (int e = 0; e < RE; ++e) {
                const float4 w = __ldg(wp[e] + i);
                wlo[e] = pack2(w.x, w.y), whi[e] = pack2(w.z, w.w);
            }
#pragma unroll
            for (int j = 0; j < TT; ++j) {
                const float4 v = XVec4<XT>::ld(xs + (size_t)j * H + 4 * i);
                const unsigned long long vlo = pack2(v.x, v.y), vhi = pack2(v.z, v.w);
#pragma unroll
                for (int e = 0; e < RE; ++e) acc[e][j] = ffma2(whi[e], vhi, ffma2(wlo[e], vlo, acc[e][j]));
            }
        }
#pragma unroll
        for (int e = 0; e < RE; ++e)
#pragma unroll
            for (int j = 0; j < TT; ++j) {
                float v = sum2(acc[e][j]);
#pragma unroll
                for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0 && t0 + j < T && r0 + e < R) lg[(size_t)(t0 + j) * ldl + r0 + e] = v;
            }
    }
}

// The same product with the roles exchanged, for many tokens: a CTA keeps WR weight rows (fp32) in shared memory and its warps stream token rows, RE per pass,
// so a token row read from L2 serves WR weight rows and the L2 reads fall from (T / 8) x |weights| to (R / WR) x |tokens|. Every logit is summed in the same
// order as in router_logits_kernel (pairs over even and odd inputs per lane, lanes combined by the same shuffles), so the two kernels agree bit for bit.
template <typename XT, int WR, int RE, int THREADS>
__global__ void __launch_bounds__(THREADS) router_logits_wres_kernel(const XT* __restrict__ x, int64_t ldx, const float* __restrict__ gw, const float* __restrict__ sgw, int T, int E,
                                                                     int H, float* __restrict__ lg, int64_t ldl) {
    extern __shared__ __align__(16) unsigned char router_smem[];
    float* ws = reinterpret_cast<float*>(router_smem);
    const int R = E + (sgw ? 1 : 0), r0 = blockIdx.x * WR, H4 = H / 4;
    for (int idx = threadIdx.x; idx < WR * H4; idx += THREADS) {
        const int e = idx / H4, c = idx - e * H4;
        const int r = min(r0 + e, R - 1);                                   // a short last group repeats its last row; the repeats are not stored
        const float* src = r < E ? gw + (size_t)r * H : sgw;
        *reinterpret_cast<float4*>(ws + (size_t)e * H + 4 * c) = __ldg(reinterpret_cast<const float4*>(src) + c);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int NW = THREADS / 32;
    for (int tg = (blockIdx.y * NW + warp) * RE; tg < T; tg += gridDim.y * NW * RE) {
        const XT* xp[RE];
#pragma unroll
        for (int j = 0; j < RE; ++j) xp[j] = x + (size_t)min(tg + j, T - 1) * ldx;   // rows past T repeat the last token; their results are not stored
        unsigned long long acc[WR][RE];
#pragma unroll
        for (int e = 0; e < WR; ++e)
#pragma unroll
            for (int j = 0; j < RE; ++j) acc[e][j] = 0ull;
        typename XVec4<XT>::Raw nxt[RE];                                    // the token chunks of the next step are in flight while this step is summed
#pragma unroll
        for (int j = 0; j < RE; ++j) nxt[j] = XVec4<XT>::ldraw(xp[j] + 4 * min(lane, H4 - 1));
        for (int i = lane; i < H4; i += 32) {
            unsigned long long vlo[RE], vhi[RE];
#pragma unroll
            for (int j = 0; j < RE; ++j) {
                const float4 v = XVec4<XT>::cvt(nxt[j]);
                vlo[j] = pack2(v.x, v.y), vhi[j] = pack2(v.z, v.w);
            }
            const int in = min(i + 32, H4 - 1);                             // past the end: a repeated load whose value is not used
#pragma unroll
            for (int j = 0; j < RE; ++j) nxt[j] = XVec4<XT>::ldraw(xp[j] + 4 * in);
#pragma unroll
            for (int e = 0; e < WR; ++e) {
                const float4 w = *reinterpret_cast<const float4*>(ws + (size_t)e * H + 4 * i);
                const unsigned long long wlo = pack2(w.x, w.y), whi = pack2(w.z, w.w);
#pragma unroll
                for (int j = 0; j < RE; ++j) acc[e][j] = ffma2(whi, vhi[j], ffma2(wlo, vlo[j], acc[e][j]));
            }
        }
#pragma unroll
        for (int j = 0; j < RE; ++j)
#pragma unroll
            for (int e = 0; e < WR; ++e) {
                float v = sum2(acc[e][j]);
#pragma unroll
                for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0 && tg + j < T && r0 + e < R) lg[(size_t)(tg + j) * ldl + r0 + e] = v;
            }
    }
}

// Rows of a grouped product that belong to no expert segment (sorted positions [*first, s): slots with an id outside the stack) are set to zero, so that
// no output row is left unwritten. A fixed small grid: the tail is empty in all but faulty inputs.
__global__ void zero_tail_rows_kernel(__half* __restrict__ d, int64_t ldd, int n, const uint32_t* __restrict__ row_map, const uint32_t* __restrict__ first, int s) {
    for (int pos = (int)*first + blockIdx.x; pos < s; pos += gridDim.x) {
        __half* row = d + (size_t)(row_map ? row_map[pos] : (uint32_t)pos) * ldd;
        for (int c = threadIdx.x; c < n; c += blockDim.x) row[c] = __float2half(0.f);
    }
}

}  // namespace kyb

int kyb_zero_tail_rows(void* d, int64_t ldd, int64_t n, const void* row_map, const void* first, int64_t s, cudaStream_t st) {
    kyb::zero_tail_rows_kernel<<<16, 256, 0, st>>>((__half*)d, ldd, (int)n, (const uint32_t*)row_map, (const uint32_t*)first, (int)s);
    return kyb_launch_check("zero_tail_rows");
}

extern "C" int kyb_moe_select(const void* logits, int64_t ld, int64_t T, int E, int K, int norm, int has_shared, void* inds, void* scs, void* sgs, void* stream) {
    KYB_REQUIRE(logits && inds && scs, "null pointer");
    KYB_REQUIRE(T > 0 && E > 0 && E <= 4096 && K > 0 && K <= 32 && K <= E, "T=%lld E=%d K=%d: need 1 <= K <= min(32, E), E <= 4096", (long long)T, E, K);
    KYB_REQUIRE(ld >= E + (has_shared ? 1 : 0), "ld=%lld is smaller than the row of logits", (long long)ld);
    KYB_REQUIRE(!has_shared || sgs, "has_shared needs the sgs output");
    const int wpb = E <= 1024 ? 4 : 1;
    const size_t smem = (size_t)wpb * E * sizeof(float);
    kyb::moe_select_kernel<<<(unsigned)((T + wpb - 1) / wpb), wpb * 32, smem, (cudaStream_t)stream>>>((const float*)logits, ld, (int)T, E, K, norm, has_shared, (uint32_t*)inds,
                                                                                                   (float*)scs, (float*)sgs);
    return kyb_launch_check("moe_select");
}

extern "C" int kyb_moe_plan(const void* ids, const void* wts, const void* rank, int E, int64_t P, int topk, int mt, void* order, void* inv, void* tok, void* ids_s,
                            void* wts_s, void* off, void* tb, void* stream) {
    KYB_REQUIRE(ids, "null pointer");
    KYB_REQUIRE(E > 0 && E <= 8192 && P > 0 && P < (1ll << 31) && topk > 0 && mt > 0, "E=%d P=%lld topk=%d mt=%d out of range", E, (long long)P, topk, mt);
    const size_t smem = (size_t)(2 * (E + 1) + 33) * sizeof(uint32_t);
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        KYB_CUDA(cudaFuncSetAttribute(kyb::moe_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((2 * 8193 + 33) * sizeof(uint32_t))));
        configured = true;
    }
    const unsigned ctas = P >= 4096 ? 8u : 1u;                                  // one cluster; 8 is the portable cluster size
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas), cfg.blockDim = dim3(kyb::PLAN_THREADS), cfg.dynamicSmemBytes = smem, cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ctas, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    const int32_t* a_ids = (const int32_t*)ids;
    const float* a_wts = (const float*)wts;
    const uint32_t* a_rank = (const uint32_t*)rank;
    int a_P = (int)P;
    uint32_t *a_order = (uint32_t*)order, *a_inv = (uint32_t*)inv, *a_tok = (uint32_t*)tok, *a_off = (uint32_t*)off, *a_tb = (uint32_t*)tb;
    int32_t* a_ids_s = (int32_t*)ids_s;
    float* a_wts_s = (float*)wts_s;
    void* args[] = {&a_ids, &a_wts, &a_rank, &E, &a_P, &topk, &mt, &a_order, &a_inv, &a_tok, &a_ids_s, &a_wts_s, &a_off, &a_tb};
    KYB_CUDA(cudaLaunchKernelExC(&cfg, (const void*)kyb::moe_plan_kernel, args));
    return kyb_launch_check("moe_plan");
}

extern "C" int kyb_gather_rows(const void* x, int64_t ldx, int64_t xrows, const void* src, int div, const void* perm, int64_t R, int64_t k, void* out, int64_t ldo,
                               void* stream) {
    KYB_REQUIRE(x && src && out && xrows > 0, "null pointer or empty source");
    KYB_REQUIRE(R > 0 && k > 0 && k % 8 == 0 && div > 0 && ldx % 8 == 0 && ldo % 8 == 0, "R=%lld k=%lld: k, ldx, ldo must be multiples of 8", (long long)R, (long long)k);
    KYB_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0, "x and out must be 16-byte aligned");
    const int64_t total = R * (k / 8);
    kyb::gather_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const __half*)x, ldx, xrows, (const uint32_t*)src, div, (const uint32_t*)perm, (int)R,
                                                                                              (int)k, (__half*)out, ldo);
    return kyb_launch_check("gather_rows");
}

extern "C" int kyb_silu_mul(const void* a, const void* b, int64_t ld, int64_t rows, int64_t n, float limit, const void* perm, void* h, int64_t ldh, void* stream) {
    KYB_REQUIRE(a && b && h, "null pointer");
    KYB_REQUIRE(rows > 0 && n > 0 && ld >= n && ldh >= n, "rows=%lld n=%lld ld=%lld ldh=%lld", (long long)rows, (long long)n, (long long)ld, (long long)ldh);
    const int64_t total = rows * n;
    if (!perm && n % 8 == 0 && ld % 8 == 0 && ldh % 8 == 0 && (((uintptr_t)a | (uintptr_t)b | (uintptr_t)h) & 15) == 0) {
        const int64_t total8 = total / 8;
        kyb::silu_mul8_kernel<<<(unsigned)((total8 + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const __half*)a, (const __half*)b, ld, total8, (int)(n / 8), limit, (__half*)h, ldh);
        return kyb_launch_check("silu_mul");
    }
    kyb::silu_mul_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const __half*)a, (const __half*)b, ld, total, (int)n, limit, (const uint32_t*)perm,
                                                                                           (__half*)h, ldh);
    return kyb_launch_check("silu_mul");
}

extern "C" int kyb_moe_combine(const void* y, int64_t ldy, const void* scs, const void* sgs, const void* shared, int64_t lds, int64_t T, int K, int64_t H, int out_dtype,
                               void* o, int64_t ldo, void* stream) {
    KYB_REQUIRE(y && scs && o, "null pointer");
    KYB_REQUIRE(T > 0 && K > 0 && H > 0 && ldy >= H && ldo >= H, "T=%lld K=%d H=%lld", (long long)T, K, (long long)H);
    KYB_REQUIRE(!shared || sgs, "a shared-expert output needs its gate values (sgs)");
    KYB_REQUIRE(out_dtype == KYB_DT_F32 || out_dtype == KYB_DT_F16, "out_dtype %d", out_dtype);
    const int64_t total = T * H;
    if (H % 8 == 0 && ldy % 8 == 0 && ldo % 8 == 0 && (!shared || lds % 8 == 0) && (((uintptr_t)y | (uintptr_t)o | (uintptr_t)shared) & 15) == 0) {
        const unsigned b8 = (unsigned)((total / 8 + 255) / 256);
        if (out_dtype == KYB_DT_F16)
            kyb::moe_combine8_kernel<__half><<<b8, 256, 0, (cudaStream_t)stream>>>((const __half*)y, ldy, (const float*)scs, (const float*)sgs, (const __half*)shared, lds, (int)T, K,
                                                                                   (int)(H / 8), (__half*)o, ldo);
        else
            kyb::moe_combine8_kernel<float><<<b8, 256, 0, (cudaStream_t)stream>>>((const __half*)y, ldy, (const float*)scs, (const float*)sgs, (const __half*)shared, lds, (int)T, K,
                                                                                  (int)(H / 8), (float*)o, ldo);
        return kyb_launch_check("moe_combine");
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dtype == KYB_DT_F16)
        kyb::moe_combine_kernel<__half><<<blocks, 256, 0, (cudaStream_t)stream>>>((const __half*)y, ldy, (const float*)scs, (const float*)sgs, (const __half*)shared, lds, (int)T, K,
                                                                                 (int)H, (__half*)o, ldo);
    else
        kyb::moe_combine_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((const __half*)y, ldy, (const float*)scs, (const float*)sgs, (const __half*)shared, lds, (int)T, K,
                                                                                (int)H, (float*)o, ldo);
    return kyb_launch_check("moe_combine");
}

template <typename XT, int TT>
static int launch_router(const void* x, int64_t ldx, const float* gw, const float* sgw, int64_t T, int E, int64_t H, float* lg, int64_t ldl, cudaStream_t st) {
    const size_t smem = (size_t)TT * (size_t)H * sizeof(XT);
    static bool configured = false;                                         // one flag per instantiation (a template static)
    if (!configured) {
        KYB_CUDA(cudaFuncSetAttribute(kyb::router_logits_kernel<XT, TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        configured = true;
    }
    const int64_t gx = (T + TT - 1) / TT;
    const int threads = T >= 1024 ? 512 : 256;                               // many tokens: 16 warps per CTA hide the L2 latency of the weight rows
    const int R = E + (sgw ? 1 : 0), ymax = (R + threads / 8 - 1) / (threads / 8);   // warps x 4 rows per pass
    const int gy = (int)std::min<int64_t>(ymax, std::max<int64_t>(1, (2 * 148 + gx - 1) / gx));   // few tokens: spread the weight rows over more CTAs
    kyb::router_logits_kernel<XT, TT><<<dim3((unsigned)gx, (unsigned)gy), threads, smem, st>>>((const XT*)x, ldx, gw, sgw, (int)T, E, (int)H, lg, ldl);
    return kyb_launch_check("router_logits");
}

static int router_sms() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        (void)cudaGetLastError();
    }
    return sms;
}

template <typename XT, int WR, int RE, int THREADS>
static int launch_router_wres(const void* x, int64_t ldx, const float* gw, const float* sgw, int64_t T, int E, int64_t H, float* lg, int64_t ldl, cudaStream_t st) {
    const size_t smem = (size_t)WR * (size_t)H * sizeof(float);
    static bool configured = false;
    if (!configured) {
        KYB_CUDA(cudaFuncSetAttribute(kyb::router_logits_wres_kernel<XT, WR, RE, THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        configured = true;
    }
    const int R = E + (sgw ? 1 : 0), gx = (R + WR - 1) / WR;
    const int64_t per_pass = (int64_t)(THREADS / 32) * RE;
    const int gy = (int)std::max<int64_t>(1, std::min<int64_t>((T + per_pass - 1) / per_pass, router_sms() / gx));   // one wave of CTAs, one CTA per SM
    kyb::router_logits_wres_kernel<XT, WR, RE, THREADS><<<dim3((unsigned)gx, (unsigned)gy), THREADS, smem, st>>>((const XT*)x, ldx, gw, sgw, (int)T, E, (int)H, lg, ldl);
    return kyb_launch_check("router_logits");
}

extern "C" int kyb_router_logits(const void* x, int x_dtype, int64_t ldx, const void* gw, const void* sgw, int64_t T, int E, int64_t H, void* lg, int64_t ldl, void* stream) {
    KYB_REQUIRE(x && gw && lg, "null pointer");
    KYB_REQUIRE(x_dtype == KYB_DT_F32 || x_dtype == KYB_DT_F16 || x_dtype == KYB_DT_BF16, "x dtype %d", x_dtype);
    KYB_REQUIRE(T > 0 && T < (1ll << 31) && E > 0 && H > 0 && H % 8 == 0 && ldx >= H && ldx % 8 == 0 && ldl >= E + (sgw ? 1 : 0), "T=%lld E=%d H=%lld: H and ldx must be multiples of 8",
                (long long)T, E, (long long)H);
    KYB_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)gw & 15) == 0 && ((uintptr_t)sgw & 15) == 0, "x, gw and sgw must be 16-byte aligned");
    const size_t per_row = (size_t)H * (x_dtype == KYB_DT_F32 ? 4 : 2);
    KYB_REQUIRE(per_row * 2 <= 226 * 1024, "H=%lld: two token rows do not fit shared memory", (long long)H);
    cudaStream_t st = (cudaStream_t)stream;
    static const bool wres = [] { const char* e = getenv("KYB_ROUTER_WRES"); return !e || atoi(e) != 0; }();   // KYB_ROUTER_WRES=0: token-resident kernel at every T
    if (wres && T >= 1024 && (size_t)H * 4 * 7 <= 226 * 1024) {            // many tokens: 7 weight rows resident per CTA, token rows streamed 8 (fp32: 4) per warp pass
        if (x_dtype == KYB_DT_F32) return launch_router_wres<float, 7, 4, 256>(x, ldx, (const float*)gw, (const float*)sgw, T, E, H, (float*)lg, ldl, st);
        if (x_dtype == KYB_DT_F16) return launch_router_wres<__half, 7, 8, 256>(x, ldx, (const float*)gw, (const float*)sgw, T, E, H, (float*)lg, ldl, st);
        return launch_router_wres<__nv_bfloat16, 7, 8, 256>(x, ldx, (const float*)gw, (const float*)sgw, T, E, H, (float*)lg, ldl, st);
    }
    const int fit = (int)((226 * 1024) / per_row);
    const int tt = (fit >= 8 && T >= 8) ? 8 : (fit >= 4 && T >= 4) ? 4 : 2;
#define KYB_ROUTER(XT)                                                                                                         \
    return tt == 8 ? launch_router<XT, 8>(x, ldx, (const float*)gw, (const float*)sgw, T, E, H, (float*)lg, ldl, st)           \
         : tt == 4 ? launch_router<XT, 4>(x, ldx, (const float*)gw, (const float*)sgw, T, E, H, (float*)lg, ldl, st)           \
                   : launch_router<XT, 2>(x, ldx, (const float*)gw, (const float*)sgw, T, E, H, (float*)lg, ldl, st)
    if (x_dtype == KYB_DT_F32) { KYB_ROUTER(float); }
    if (x_dtype == KYB_DT_F16) { KYB_ROUTER(__half); }
    KYB_ROUTER(__nv_bfloat16);
#undef KYB_ROUTER
}

// ---- tensor-core router (prefill): kyb_router_split once per gate, kyb_router_logits_tc per call.
// pieces: fp16 [3 * rpad, H] with rpad = kyb_router_rpad(E, shared) (rows rounded up to 8); inv_scale: float [rpad].
extern "C" int64_t kyb_router_rpad(int E, int has_shared) { return ((int64_t)E + (has_shared ? 1 : 0) + 7) / 8 * 8; }

extern "C" int kyb_router_split(const void* gw, const void* sgw, int E, int64_t H, void* pieces, void* inv_scale, void* stream) {
    KYB_REQUIRE(gw && pieces && inv_scale, "null pointer");
    KYB_REQUIRE(E > 0 && H > 0 && H < (1ll << 31), "E=%d H=%lld", E, (long long)H);
    const int R = E + (sgw ? 1 : 0), rpad = (int)kyb_router_rpad(E, sgw != nullptr);
    kyb::router_split_kernel<<<(unsigned)rpad, 256, 0, (cudaStream_t)stream>>>((const float*)gw, (const float*)sgw, E, R, rpad, (int)H, (__half*)pieces, (float*)inv_scale);
    return kyb_launch_check("router_split");
}

// lg fp32 [T, >= R] = x fp16 [T, H] on the gate whose pieces were made by kyb_router_split (R = E + has_shared columns are written). work: float [T, 3 rpad]
// (16-byte aligned), the partial products of the three pieces. Replaces the fp32 contraction of kyojin_mlx/foreign_moe.py:122-130 for many tokens: the products
// run on tcgen05 (fp16 x fp16 -> fp32, exact products), one more launch recombines them.
extern "C" int kyb_router_logits_tc(const void* x, int64_t ldx, const void* pieces, const void* inv_scale, int64_t T, int E, int has_shared, int64_t H, void* work,
                                    void* lg, int64_t ldl, void* stream) {
    KYB_REQUIRE(x && pieces && inv_scale && work && lg, "null pointer");
    const int R = E + (has_shared ? 1 : 0), rpad = (int)kyb_router_rpad(E, has_shared);
    KYB_REQUIRE(T > 0 && T < (1ll << 31) && E > 0 && H > 0 && H % 64 == 0 && ldx >= H && ldx % 8 == 0 && ldl >= R, "T=%lld E=%d H=%lld: H must be a multiple of 64", (long long)T, E,
                (long long)H);
    if (int rc = kyb_gemm_f16_tn_f32(x, ldx, pieces, H, T, 3 * (int64_t)rpad, H, 1.0f, work, 3 * (int64_t)rpad, stream)) return rc;
    const int64_t total = T * R;
    kyb::router_combine_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const float*)work, 3 * (int64_t)rpad, (const float*)inv_scale, (int)T, R, rpad,
                                                                                                  (float*)lg, ldl);
    return kyb_launch_check("router_combine");
}
