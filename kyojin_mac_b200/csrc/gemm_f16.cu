// Prefill GEMM on tcgen05: D[m, n] = sat_f16(gscale * sum_k A[m, k] * B[n, k]) with fp16 operands and fp32 accumulation in tensor memory.
// A = activations [M, K], B = dequantised weights [N, K] (fp16 exactly as the reference stages them: kyojin_mlx/foreign_metal.py:1130-1146),
// both K-major, so this is the x W^T contraction of kyojin_mlx/foreign_linear.py:710/:737 (`x2 @ self.dequant().T`).
//
// Persistent CTAs (one per SM) walk over 128 x BN output tiles. Warp 0 feeds a ring of shared-memory stages with TMA tiled loads (128-byte swizzle), warp 1 issues
// tcgen05.mma (UMMA 128 x BN x 16, kind::f16) from one elected thread and hands stages back through tcgen05.commit, warps 2-5 read the accumulator
// from tensor memory with tcgen05.ld and store fp16 rows. Every mbarrier wait is bounded: a wait that gives up sets the device status word and
// the CTA drains and frees its tensor memory.
#include <algorithm>
#include <mutex>
#include <unordered_map>

#include "tc_common.cuh"

namespace kyb {

constexpr int GM_BM = 128, GM_BK = 64, GM_THREADS = 192;

struct GemmParams {
    __half* d;
    float* d32;                // when set, the epilogue stores gscale * accumulator as fp32 here (unsaturated) instead of fp16 at d
    int64_t ldd;
    int m, n, k;
    float gscale;
    unsigned int* status;
    // grouped mode (routed experts, rows of A sorted by expert): tile blockIdx.y belongs to the expert e with tb[e] <= tile < tb[e + 1]; its rows start at
    // off[e] + (tile - tb[e]) * 128 and end at off[e + 1]; B rows of expert e start at e * n. row_map (optional) scatters output rows.
    const uint32_t* tb;
    const uint32_t* off;
    const uint32_t* row_map;
    const float* gs;           // per-expert output scale or null
    int experts;
    int tiles_m;               // dense mode: tile rows; consecutive tiles walk down m first (the activations stay in L2 while each weight tile is streamed once)
};

// What one output tile covers (dense: a 128 x BN block of D; grouped: 128 rows of one expert's segment)
struct TileInfo {
    int m0, m_end, n0, b_row0;
    float gscale;
    bool valid;
};

template <int BN>
__device__ __forceinline__ TileInfo tile_info(const GemmParams& p, int t, int tiles_n) {
    TileInfo ti;
    const int tn = p.tb ? t % tiles_n : t / p.tiles_m, tm = p.tb ? t / tiles_n : t % p.tiles_m;
    ti.n0 = tn * BN, ti.m0 = tm * GM_BM, ti.m_end = p.m, ti.b_row0 = ti.n0, ti.gscale = p.gscale, ti.valid = true;
    if (p.tb) {
        if ((uint32_t)tm >= p.tb[p.experts]) {
            ti.valid = false;
            return ti;
        }
        int lo = 0, hi = p.experts;                                                 // largest e with tb[e] <= tm (empty experts repeat a value)
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (p.tb[mid] <= (uint32_t)tm) lo = mid; else hi = mid;
        }
        ti.m0 = (int)(p.off[lo] + ((uint32_t)tm - p.tb[lo]) * GM_BM);
        ti.m_end = (int)p.off[lo + 1];
        ti.b_row0 = lo * p.n + ti.n0;
        if (p.gs) ti.gscale = p.gs[lo];
    }
    return ti;
}

// Persistent: CTA c works on tiles c, c + gridDim.x, ... Two accumulators (2 x BN tensor-memory columns) alternate, so the epilogue of one tile overlaps
// the MMAs of the next.
template <int BN, int STAGES>
__global__ void __launch_bounds__(GM_THREADS, 1) gemm_f16_tn_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const GemmParams p,
                                                                    const int tiles_n, const int num_tiles) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr uint32_t A_BYTES = GM_BM * GM_BK * 2, B_BYTES = BN * GM_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;                 // 1024-byte alignment for the 128-byte swizzle atoms
    const uint32_t bars = smem0 + STAGES * STAGE_BYTES;                            // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], tmem slot
    const uint32_t full0 = bars, empty0 = bars + 8 * STAGES, accf0 = bars + 16 * STAGES, acce0 = accf0 + 16, tmem_slot = acce0 + 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = p.k / GM_BK;
    constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init_a(full0 + 8 * s, 1), mbar_init_a(empty0 + 8 * s, 1);
        for (int a = 0; a < 2; ++a) mbar_init_a(accf0 + 8 * a, 1), mbar_init_a(acce0 + 8 * a, 4);
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
        // ---- TMA producer
        if (elect_one()) {
            uint32_t parity = 1;                                                    // a fresh barrier passes a wait on the previous phase
            int s = 0;
            for (int t = blockIdx.x; t < num_tiles && !failed; t += gridDim.x) {
                const TileInfo ti = tile_info<BN>(p, t, tiles_n);
                if (!ti.valid) continue;
                for (int kb = 0; kb < kblocks && !failed; ++kb) {
                    if (!mbar_wait_fast(empty0 + 8 * s, parity)) failed = true;
                    const uint32_t a_dst = smem0 + s * STAGE_BYTES, b_dst = a_dst + A_BYTES;
                    mbar_expect_tx_a(full0 + 8 * s, STAGE_BYTES);
                    tma_load_2d(a_dst, &tma_a, kb * GM_BK, ti.m0, full0 + 8 * s);
                    tma_load_2d(b_dst, &tma_b, kb * GM_BK, ti.b_row0, full0 + 8 * s);
                    if (++s == STAGES) s = 0, parity ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (elect_one()) {
            constexpr uint32_t idesc = umma_idesc_f16(GM_BM, BN);
            uint32_t parity = 0;
            int s = 0, it = 0;
            for (int t = blockIdx.x; t < num_tiles && !failed; t += gridDim.x) {
                if (!tile_info<BN>(p, t, tiles_n).valid) continue;
                const int acc = it & 1;
                if (!mbar_wait_fast(acce0 + 8 * acc, (((uint32_t)it >> 1) & 1u) ^ 1u)) failed = true;      // the epilogue has drained this accumulator
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < kblocks && !failed; ++kb) {
                    if (!mbar_wait_fast(full0 + 8 * s, parity)) failed = true;
                    tc_fence_after();
                    const uint64_t adesc = umma_desc_sw128(smem0 + s * STAGE_BYTES), bdesc = umma_desc_sw128(smem0 + s * STAGE_BYTES + A_BYTES);
#pragma unroll
                    for (int kk = 0; kk < GM_BK / 16; ++kk)                         // 16 fp16 = 32 bytes along K inside the swizzle atom: +2 in the address field
                        umma_f16(tmem_d, adesc + 2 * kk, bdesc + 2 * kk, idesc, (kb | kk) != 0);
                    umma_commit(empty0 + 8 * s);                                    // stage free once these MMAs have read it
                    if (++s == STAGES) s = 0, parity ^= 1u;
                }
                umma_commit(accf0 + 8 * acc);                                       // accumulator complete
                ++it;
            }
        }
    } else {
        // ---- epilogue: warp w may touch TMEM lanes [32 (w % 4), 32 (w % 4) + 32)
        const int q = warp & 3;
        int it = 0;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
            const TileInfo ti = tile_info<BN>(p, t, tiles_n);
            if (!ti.valid) continue;
            const int acc = it & 1;
            if (!mbar_wait_fast(accf0 + 8 * acc, ((uint32_t)it >> 1) & 1u)) failed = true;
            tc_fence_after();
            const int row = ti.m0 + q * 32 + lane;
            const size_t orow = (p.row_map && row < ti.m_end) ? (size_t)p.row_map[row] : (size_t)row;
            __half* drow = p.d + orow * p.ldd + ti.n0;
            float* frow = p.d32 + orow * p.ldd + ti.n0;
            const float gscale = ti.gscale;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c), v);
                tmem_ld_wait();
                if (p.d32) {
                    if (row < ti.m_end && !failed) {
                        if (ti.n0 + c + 32 <= p.n && (p.ldd & 3) == 0) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                *reinterpret_cast<float4*>(frow + c + j) = make_float4(__uint_as_float(v[j]) * gscale, __uint_as_float(v[j + 1]) * gscale,
                                                                                       __uint_as_float(v[j + 2]) * gscale, __uint_as_float(v[j + 3]) * gscale);
                        } else {
                            for (int j = 0; j < 32; ++j)
                                if (ti.n0 + c + j < p.n) frow[c + j] = __uint_as_float(v[j]) * gscale;
                        }
                    }
                } else if (row < ti.m_end && !failed) {
                    if (ti.n0 + c + 32 <= p.n && (p.ldd & 7) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint4 o;
                            __half2 h0 = sat_half2(__uint_as_float(v[j]) * gscale, __uint_as_float(v[j + 1]) * gscale);
                            __half2 h1 = sat_half2(__uint_as_float(v[j + 2]) * gscale, __uint_as_float(v[j + 3]) * gscale);
                            __half2 h2 = sat_half2(__uint_as_float(v[j + 4]) * gscale, __uint_as_float(v[j + 5]) * gscale);
                            __half2 h3 = sat_half2(__uint_as_float(v[j + 6]) * gscale, __uint_as_float(v[j + 7]) * gscale);
                            o.x = *reinterpret_cast<uint32_t*>(&h0), o.y = *reinterpret_cast<uint32_t*>(&h1), o.z = *reinterpret_cast<uint32_t*>(&h2), o.w = *reinterpret_cast<uint32_t*>(&h3);
                            *reinterpret_cast<uint4*>(drow + c + j) = o;
                        }
                    } else {
                        for (int j = 0; j < 32; ++j)
                            if (ti.n0 + c + j < p.n) drow[c + j] = sat_half(__uint_as_float(v[j]) * gscale);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_a(acce0 + 8 * acc);                          // this warp has read its quarter of the accumulator
            ++it;
        }
    }
    if (failed) atomicExch(p.status, KYB_DEV_TIMEOUT_GEMM);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace kyb

namespace {

template <int BN, int STAGES>
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const kyb::GemmParams& p, cudaStream_t st, int tiles_y) {
    constexpr size_t smem = (size_t)STAGES * (kyb::GM_BM * kyb::GM_BK * 2 + BN * kyb::GM_BK * 2) + 16 * STAGES + 48 + 1024;
    auto kern = kyb::gemm_f16_tn_kernel<BN, STAGES>;
    static std::mutex mu;
    static unsigned done = 0;
    static int sms = 0;
    int dev = 0;
    KYB_CUDA(cudaGetDevice(&dev));
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!(done & (1u << (dev & 31)))) {
            KYB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            done |= 1u << (dev & 31);
        }
        if (!sms) KYB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    }
    const int tiles_n = (p.n + BN - 1) / BN;
    const int tiles_m = tiles_y ? tiles_y : (p.m + kyb::GM_BM - 1) / kyb::GM_BM;
    const int num_tiles = tiles_n * tiles_m;
    kyb::GemmParams pp = p;
    pp.tiles_m = tiles_m;
    kern<<<(unsigned)std::min(num_tiles, sms), kyb::GM_THREADS, smem, st>>>(ta, tb, pp, tiles_n, num_tiles);
    return kyb_launch_check("gemm_f16_tn");
}

}  // namespace

// D fp16 [m, n] (row stride ldd) = sat(gscale * A [m, k] (row stride lda) x B [n, k]^T (row stride ldb)), all fp16, k % 64 == 0.
extern "C" int kyb_gemm_f16_tn(const void* a, int64_t lda, const void* b, int64_t ldb, int64_t m, int64_t n, int64_t k, float gscale, void* d, int64_t ldd,
                               void* stream) {
    KYB_REQUIRE(a && b && d, "null pointer");
    KYB_REQUIRE(m > 0 && n > 0 && k > 0 && k % 64 == 0, "m=%lld n=%lld k=%lld: k must be a positive multiple of 64", (long long)m, (long long)n, (long long)k);
    KYB_REQUIRE(lda >= k && ldb >= k && lda % 8 == 0 && ldb % 8 == 0 && ldd >= n, "leading dimensions: lda, ldb >= k and multiples of 8, ldd >= n");
    KYB_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)b & 15) == 0 && ((uintptr_t)d & 1) == 0, "a and b must be 16-byte aligned");
    KYB_REQUIRE(m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 31), "dimension too large");
    unsigned int* status = kyb_device_status_word();
    KYB_REQUIRE(status, "could not set up the device status word");
    const bool wide = n >= 256;
    CUtensorMap ta, tb;
    if (int rc = kyb_make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a, (uint64_t)m, (uint64_t)k, (uint64_t)lda * 2, kyb::GM_BM, kyb::GM_BK)) return rc;
    if (int rc = kyb_make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, b, (uint64_t)n, (uint64_t)k, (uint64_t)ldb * 2, wide ? 256 : 128, kyb::GM_BK)) return rc;
    kyb::GemmParams p;
    p.d = (__half*)d, p.d32 = nullptr, p.ldd = ldd, p.m = (int)m, p.n = (int)n, p.k = (int)k, p.gscale = gscale, p.status = status;
    p.tb = nullptr, p.off = nullptr, p.row_map = nullptr, p.gs = nullptr, p.experts = 0;
    cudaStream_t st = (cudaStream_t)stream;
    return wide ? launch_gemm<256, 4>(ta, tb, p, st, 0) : launch_gemm<128, 6>(ta, tb, p, st, 0);
}

// The same product with the fp32 accumulators written out unrounded: d fp32 [m, n] (row stride ldd floats) = gscale * A x B^T. Used where the fp16 operands are
// exact pieces of wider numbers and the caller recombines the partial products (the tensor-core router, csrc/moe.cu).
extern "C" int kyb_gemm_f16_tn_f32(const void* a, int64_t lda, const void* b, int64_t ldb, int64_t m, int64_t n, int64_t k, float gscale, void* d, int64_t ldd,
                                   void* stream) {
    KYB_REQUIRE(a && b && d, "null pointer");
    KYB_REQUIRE(m > 0 && n > 0 && k > 0 && k % 64 == 0, "m=%lld n=%lld k=%lld: k must be a positive multiple of 64", (long long)m, (long long)n, (long long)k);
    KYB_REQUIRE(lda >= k && ldb >= k && lda % 8 == 0 && ldb % 8 == 0 && ldd >= n, "leading dimensions: lda, ldb >= k and multiples of 8, ldd >= n");
    KYB_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)b & 15) == 0 && ((uintptr_t)d & 15) == 0, "a, b and d must be 16-byte aligned");
    KYB_REQUIRE(m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 31), "dimension too large");
    unsigned int* status = kyb_device_status_word();
    KYB_REQUIRE(status, "could not set up the device status word");
    const bool wide = n >= 256;
    CUtensorMap ta, tb;
    if (int rc = kyb_make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a, (uint64_t)m, (uint64_t)k, (uint64_t)lda * 2, kyb::GM_BM, kyb::GM_BK)) return rc;
    if (int rc = kyb_make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, b, (uint64_t)n, (uint64_t)k, (uint64_t)ldb * 2, wide ? 256 : 128, kyb::GM_BK)) return rc;
    kyb::GemmParams p;
    p.d = nullptr, p.d32 = (float*)d, p.ldd = ldd, p.m = (int)m, p.n = (int)n, p.k = (int)k, p.gscale = gscale, p.status = status;
    p.tb = nullptr, p.off = nullptr, p.row_map = nullptr, p.gs = nullptr, p.experts = 0;
    cudaStream_t st = (cudaStream_t)stream;
    return wide ? launch_gemm<256, 4>(ta, tb, p, st, 0) : launch_gemm<128, 6>(ta, tb, p, st, 0);
}

// Grouped form for routed experts: a fp16 [s, k] rows sorted by expert (segment e = rows [off[e], off[e + 1])), b fp16 [experts * n, k] (expert stack),
// tb / off from kyb_moe_plan with mt = 128, row_map (optional, u32 [s]) = output row of each sorted row, gs (optional) per-expert output scale.
// d [*, n]. The grid is sized for the worst case (s / 128 + experts tiles); tiles past tb[experts] exit at once.
extern "C" int kyb_gemm_f16_grouped(const void* a, int64_t lda, const void* b, int64_t ldb, int64_t s, int64_t n, int64_t k, int experts, const void* tb_, const void* off,
                                    const void* row_map, const void* gs, void* d, int64_t ldd, void* stream) {
    KYB_REQUIRE(a && b && d && tb_ && off, "null pointer");
    KYB_REQUIRE(s > 0 && n > 0 && k > 0 && k % 64 == 0 && experts > 0, "s=%lld n=%lld k=%lld experts=%d: k must be a positive multiple of 64", (long long)s, (long long)n,
                (long long)k, experts);
    KYB_REQUIRE(n % 128 == 0, "grouped GEMM needs n %% 128 == 0 (an output tile must not straddle two experts), got n=%lld", (long long)n);
    KYB_REQUIRE(lda >= k && ldb >= k && lda % 8 == 0 && ldb % 8 == 0 && ldd >= n, "leading dimensions: lda, ldb >= k and multiples of 8, ldd >= n");
    KYB_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)b & 15) == 0, "a and b must be 16-byte aligned");
    unsigned int* status = kyb_device_status_word();
    KYB_REQUIRE(status, "could not set up the device status word");
    const bool wide = n % 256 == 0;
    CUtensorMap ta, tb;
    if (int rc = kyb_make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a, (uint64_t)s, (uint64_t)k, (uint64_t)lda * 2, kyb::GM_BM, kyb::GM_BK)) return rc;
    if (int rc = kyb_make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, b, (uint64_t)experts * (uint64_t)n, (uint64_t)k, (uint64_t)ldb * 2, wide ? 256 : 128, kyb::GM_BK)) return rc;
    kyb::GemmParams p;
    p.d = (__half*)d, p.d32 = nullptr, p.ldd = ldd, p.m = (int)s, p.n = (int)n, p.k = (int)k, p.gscale = 1.0f, p.status = status;
    p.tb = (const uint32_t*)tb_, p.off = (const uint32_t*)off, p.row_map = (const uint32_t*)row_map, p.gs = (const float*)gs, p.experts = experts;
    const int max_tiles = (int)((s + kyb::GM_BM - 1) / kyb::GM_BM) + experts;
    cudaStream_t st = (cudaStream_t)stream;
    if (int rc = wide ? launch_gemm<256, 4>(ta, tb, p, st, max_tiles) : launch_gemm<128, 6>(ta, tb, p, st, max_tiles)) return rc;
    return kyb_zero_tail_rows(d, ldd, n, row_map, (const uint32_t*)off + experts, s, st);                      // slots that belong to no expert: rows of zeros
}
