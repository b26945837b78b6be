// tcgen05 / TMA building blocks shared by the prefill GEMM kernels (sm_100a): tensor-map encoding on the host, bulk-tensor loads, UMMA
// shared-memory and instruction descriptors, TMEM allocation, commit / fence / load wrappers. All device-side waits are bounded.
#pragma once

#include <cuda.h>

#include "kyb_common.cuh"

// ------------------------------------------------------------------------------------------------ host: tensor maps
// cuTensorMapEncodeTiled is fetched through the runtime's driver entry point lookup, so the library has no link-time dependency on libcuda.
typedef CUresult (*kyb_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                        const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline kyb_encode_tiled_fn kyb_get_encode_tiled() {
    static kyb_encode_tiled_fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (kyb_encode_tiled_fn)p;
    }
    return fn;
}

// 2-D row-major tensor [rows, cols] of `elem_bytes`-wide elements, row stride `ld_bytes`; box [box_rows, box_cols]; 128-byte swizzle by default
// (box_cols * elem_bytes must equal the swizzle width). Out-of-range parts of a box are filled with zeros on loads and dropped on stores.
static inline int kyb_make_tmap_2d(CUtensorMap* tm, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_bytes,
                                   uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
    kyb_encode_tiled_fn enc = kyb_get_encode_tiled();
    if (!enc) {
        kyb_set_error("cuTensorMapEncodeTiled is not available from this driver");
        return KYB_ECUDA;
    }
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    (void)elem_bytes;
    const CUresult r = enc(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        kyb_set_error("cuTensorMapEncodeTiled failed with CUresult %d (base %p rows %llu cols %llu ld %llu box %u x %u)", (int)r, base, (unsigned long long)rows,
                      (unsigned long long)cols, (unsigned long long)ld_bytes, box_rows, box_cols);
        return KYB_ECUDA;
    }
    return KYB_OK;
}

// Tensor maps of the output matrix on every receiving rank (one entry without sharding): 16-bit elements, box 32 rows x 32 columns, 64-byte swizzle.
struct KybOutMaps {
    CUtensorMap m[8];
};
constexpr uint32_t KYB_STG_BYTES = 2048;    // epilogue staging per warp: 32 rows x 32 16-bit columns

#ifdef __CUDACC__
namespace kyb {

// ------------------------------------------------------------------------------------------------ device: TMA tiled load
// x (innermost coordinate) must keep x * elem_bytes a multiple of 16; callers pass multiples of the 128-byte box width.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst), "l"(tm), "r"(x), "r"(y),
                 "r"(bar)
                 : "memory");
}
// shared -> global tiled store (bulk async group of the issuing thread); x * elem_bytes must be a multiple of 16, coordinates must not be negative
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(tm), "r"(x), "r"(y), "r"(src) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }   // the sources of this thread's stores have been read
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }          // this thread's stores are complete
// Epilogue step of one warp: 32 rows (one per lane) x 32 columns given as 16 packed pairs w[16] go to the warp's staging buffer (64-byte swizzle, conflict-free
// 16-byte stores) and leave as one tiled bulk store per receiving rank at (x, y); rows / columns outside the matrix are dropped by the tensor map.
__device__ __forceinline__ void epilogue_stage_store(const KybOutMaps& outs, int nout, uint32_t stg, int lane, const uint32_t (&w)[16], int x, int y, bool issue) {
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");      // the previous step's stores have read the staging buffer
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 4; ++j)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stg + (uint32_t)lane * 64u + (uint32_t)((j ^ ((lane >> 1) & 3)) << 4)), "r"(w[4 * j]), "r"(w[4 * j + 1]),
                     "r"(w[4 * j + 2]), "r"(w[4 * j + 3])
                     : "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0 && issue) {
        for (int pr = 0; pr < nout; ++pr)
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(&outs.m[pr]), "r"(x), "r"(y), "r"(stg) : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
}
// Wide form for outputs that also go to other GPUs: two 32-column steps (half = 0, then 1) fill a [32 rows][128 bytes] buffer (128-byte swizzle; 4 KB, 1024-byte
// aligned) and leave as one tiled bulk store of 32 x 64 columns per receiving rank: full 128-byte row segments on NVLink instead of 64-byte ones.
__device__ __forceinline__ void epilogue_stage_store_wide(const KybOutMaps& outs, int nout, uint32_t stg, int lane, const uint32_t (&w)[16], int half, int x, int y, bool issue) {
    if (half == 0) {
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stg + (uint32_t)lane * 128u + (uint32_t)(((j + 4 * half) ^ (lane & 7)) << 4)), "r"(w[4 * j]), "r"(w[4 * j + 1]),
                     "r"(w[4 * j + 2]), "r"(w[4 * j + 3])
                     : "memory");
    if (half == 1) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0 && issue) {
            for (int pr = 0; pr < nout; ++pr)
                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(&outs.m[pr]), "r"(x), "r"(y), "r"(stg) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
    }
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* tm) { asm volatile("prefetch.tensormap [%0];" ::"l"(tm) : "memory"); }

__device__ __forceinline__ void mbar_init_a(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory"); }
__device__ __forceinline__ void mbar_expect_tx_a(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_a(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }

// ------------------------------------------------------------------------------------------------ device: UMMA descriptors
// K-major operand tile in shared memory written with the 128-byte swizzle (rows of 128 bytes, 8-row groups of 1024 bytes, base 1024-aligned):
// start address >> 4 in bits [0,14), leading byte offset (unused for swizzled K-major, set to 1) in [16,30), stride byte offset = 1024 >> 4 in
// [32,46), descriptor version 1 in [46,48), layout type SWIZZLE_128B = 2 in [61,64).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// kind::f16 instruction descriptor: D = f32 (1 << 4), A = B = f16 (format 0), both K-major, N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t umma_idesc_f16(int m, int n) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24); }

// D[tmem] (+)= A[smem] * B[smem]^T, issued by one thread
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// mbarrier arrive once every tcgen05 operation issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// TMEM: `cols` (power of two >= 32) columns; the base address is written to shared memory at `dst`. Executed by one whole warp.
__device__ __forceinline__ void tmem_alloc(uint32_t dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) { asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory"); }

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives row (lane base + i), columns [col, col + 32)
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]),
          "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------------------------------------------ device: CTA pairs (tcgen05 cta_group::2)
// A cluster of two CTAs on neighbouring SMs shares one MMA: each holds its own rows of the M-side operand and half of the N-side operand, the leader (cluster rank
// 0) issues the instruction for both tensor cores. Loads of either CTA complete on a barrier of the leader (cta_group::2 form of the tiled load, the barrier given
// by its shared::cluster address; no multicast load), tcgen05.commit signals the barrier at one offset in both CTAs.
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// tiled load into this CTA's shared memory whose bytes complete on a barrier of the pair's leader (bar: shared::cluster address)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* tm, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst), "l"(tm), "r"(x),
                 "r"(y), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) { asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) { asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory"); }
// arrives on the barrier at this offset in both CTAs of the pair once every tcgen05 operation issued so far by this thread has completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"((unsigned short)3) : "memory");
}

// arrival on a barrier of the other CTA of the pair (bar: shared::cluster address), default semantics (release at CTA scope)
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

}  // namespace kyb
#endif
