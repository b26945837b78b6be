// Shared host/device helpers of the kyb library: status plumbing, bounded mbarrier waits, bulk copies, mma.sync wrappers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/kyb.h"

// ------------------------------------------------------------------------------------------------ host side
void kyb_set_error(const char* fmt, ...);
unsigned int* kyb_device_status_word();   // per-device word in global memory, zero-initialised (nullptr on failure)
// grouped products: zero the output rows of the sorted positions [*first, s) (slots that belong to no expert segment); first = device pointer to off[E]
int kyb_zero_tail_rows(void* d, int64_t ldd, int64_t n, const void* row_map, const void* first, int64_t s, cudaStream_t st);

#define KYB_REQUIRE(cond, ...)                                        \
    do {                                                              \
        if (!(cond)) {                                                \
            kyb_set_error(__VA_ARGS__);                               \
            return KYB_EINVAL;                                        \
        }                                                             \
    } while (0)

#define KYB_CUDA(call)                                                                           \
    do {                                                                                         \
        cudaError_t e__ = (call);                                                                \
        if (e__ != cudaSuccess) {                                                                \
            kyb_set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), __FILE__, __LINE__); \
            return KYB_ECUDA;                                                                    \
        }                                                                                        \
    } while (0)

static inline int kyb_launch_check(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        kyb_set_error("launch of %s failed: %s", what, cudaGetErrorString(e));
        return KYB_ECUDA;
    }
    return KYB_OK;
}

// T16 tile geometry (kyojin_mac_b200/layout.py holds the layout description)
__host__ __device__ constexpr int kyb_tile_bytes(int fmt) {
    return fmt == KYB_FMT_Q4_K ? 2304 : fmt == KYB_FMT_Q6_K ? 3360 : fmt == KYB_FMT_Q3_K ? 1760 : fmt == KYB_FMT_Q5_K ? 2816 : fmt == KYB_FMT_Q8_0 ? 4352 : fmt == KYB_FMT_Q2_K ? 1344 : fmt == KYB_FMT_IQ4_XS ? 2176 : 2304;
}
__host__ __device__ constexpr int kyb_raw_block_elems(int fmt) { return fmt == KYB_FMT_NVFP4 ? 64 : fmt == KYB_FMT_Q8_0 ? 32 : 256; }
__host__ __device__ constexpr int kyb_raw_block_bytes(int fmt) {
    return fmt == KYB_FMT_Q4_K ? 144 : fmt == KYB_FMT_Q6_K ? 210 : fmt == KYB_FMT_Q3_K ? 110 : fmt == KYB_FMT_Q5_K ? 176 : fmt == KYB_FMT_Q8_0 ? 34 : fmt == KYB_FMT_Q2_K ? 84 : fmt == KYB_FMT_IQ4_XS ? 136 : 36;
}
// stored bytes of one 256-input block of a row (NVFP4: four 36-byte blocks, Q8_0: eight 34-byte blocks)
__host__ __device__ constexpr int kyb_raw_kblock_bytes(int fmt) { return 256 / kyb_raw_block_elems(fmt) * kyb_raw_block_bytes(fmt); }
// formats whose blocks carry per-sub-block minima (w = d sc q - dmin mn): the GEMV subtracts them through staged sums of x
__host__ __device__ constexpr bool kyb_has_mins(int fmt) { return fmt == KYB_FMT_Q4_K || fmt == KYB_FMT_Q5_K; }
// Q2_K: one 4-bit minimum per 16 inputs (16 per block): the staged sums are per 16 inputs
__host__ __device__ constexpr bool kyb_has_mins16(int fmt) { return fmt == KYB_FMT_Q2_K; }

// status codes written to the device status word by kernels whose bounded wait expired
#define KYB_DEV_TIMEOUT_GEMV 0x1001u
#define KYB_DEV_TIMEOUT_GEMM 0x1002u
#define KYB_DEV_TIMEOUT_SELFTEST 0x10FFu

#ifdef __CUDACC__
// ------------------------------------------------------------------------------------------------ device side
namespace kyb {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_a_local(uint32_t bar) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: every try_wait already blocks for a hardware-defined slice; after `limit` failed slices the caller
// gives up (the kernel then records a status and drains). Returns true when the phase completed.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 22)) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(64);
    }
    return false;
}

// The same by shared address, with the common case (data already there) inline and the polling loop out of line.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (i > 64) __nanosleep(64);
    }
    return false;
}
__device__ __forceinline__ bool mbar_wait_fast(uint32_t bar, uint32_t parity, uint32_t limit = (1u << 22)) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    return mbar_wait_slow(bar, parity, limit);
}

// 1-D bulk copy global -> this CTA's shared memory, completion counted in bytes on `bar`.
// dst, src 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes),
                 "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bulk_g2s_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(smem_u32(dst)), "l"(src),
                 "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// D(16x8, f32) += A(16x16, f16 row) * B(16x8, f16 col)
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t a0, const uint32_t a1, const uint32_t a2, const uint32_t a3, const uint32_t b0,
                                         const uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D(16x8, f32) = A(16x16, f16 row) * B(16x8, f16 col)   (zero accumulator input: no register initialisation needed)
__device__ __forceinline__ void mma16816_z(float (&d)[4], const uint32_t a0, const uint32_t a1, const uint32_t a2, const uint32_t a3, const uint32_t b0,
                                           const uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ void mma1688_z(float (&d)[4], const uint32_t a0, const uint32_t a1, const uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "f"(0.f));
}
// D(16x8, f32) += A(16x8, f16 row) * B(8x8, f16 col)
__device__ __forceinline__ void mma1688(float (&d)[4], const uint32_t a0, const uint32_t a1, const uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}

// shared-memory accesses by 32-bit shared-window address (keeps address arithmetic in one 32-bit register with immediate offsets)
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t a) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts128f(uint32_t a, float4 v) {
    asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(a), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
// (a & mask) | b   in one LOP3
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t b) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(b));   // (a & b) | c
    return r;
}

__device__ __forceinline__ float half_bits_to_float(uint32_t h16) { return __half2float(__ushort_as_half((unsigned short)h16)); }

// float -> fp16, round to nearest even, saturated to +-65504 (infinities too); NaN stays NaN. One conversion instruction: the same bits as clamping first and
// converting after for every input that is not a NaN (a clamp built from fminf / fmaxf would turn a NaN into -65504).
__device__ __forceinline__ __half sat_half(float v) {
    unsigned short d;
    asm("cvt.rn.satfinite.f16.f32 %0, %1;" : "=h"(d) : "f"(v));
    return __ushort_as_half(d);
}
// two at once: (lo, hi) -> packed pair
__device__ __forceinline__ __half2 sat_half2(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return *reinterpret_cast<__half2*>(&d);
}

}  // namespace kyb
#endif
