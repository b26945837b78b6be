// Status plumbing of the kyb C ABI: thread-local error text, status strings, the per-device status word.
#include <stdarg.h>
#include <string.h>

#include <mutex>

#include "kyb_common.cuh"

static thread_local char g_err[512] = "";

void kyb_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

// The status word is part of the library image (zero-initialised on every device that loads it), so no entry point allocates device memory.
static __device__ __align__(256) unsigned int g_status_word_dev[64];
static std::mutex g_status_mu;
static unsigned int* g_status_words[64] = {nullptr};

unsigned int* kyb_device_status_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(g_status_mu);
    if (!g_status_words[dev]) {
        void* p = nullptr;                                             // the symbol's address on the current device (the name itself is a host-side stand-in)
        if (cudaGetSymbolAddress(&p, g_status_word_dev) != cudaSuccess) return nullptr;
        g_status_words[dev] = (unsigned int*)p;
    }
    return g_status_words[dev];
}

extern "C" {

int kyb_version(void) { return 100; }

const char* kyb_status_string(int status) {
    switch (status) {
        case KYB_OK: return "ok";
        case KYB_EINVAL: return "invalid argument";
        case KYB_ECUDA: return "CUDA runtime error";
        case KYB_ETIMEOUT: return "a bounded device-side wait expired";
        case KYB_EUNSUPPORTED: return "unsupported request";
        case KYB_EWORKSPACE: return "workspace missing or too small";
        default: return "unknown status";
    }
}

const char* kyb_last_error(void) { return g_err; }

int kyb_check_device_status(void* stream) {
    unsigned int* w = kyb_device_status_word();
    if (!w) {
        kyb_set_error("no device status word (no CUDA device?)");
        return KYB_ECUDA;
    }
    unsigned int v = 0;
    KYB_CUDA(cudaMemcpyAsync(&v, w, sizeof(v), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    KYB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (v) {
        KYB_CUDA(cudaMemsetAsync(w, 0, sizeof(v), (cudaStream_t)stream));
        kyb_set_error("device status 0x%x: a kernel gave up a bounded wait", v);
        return KYB_ETIMEOUT;
    }
    return KYB_OK;
}

size_t kyb_t16_nbytes(int fmt, int64_t n, int64_t k) {
    if (fmt < 0 || fmt >= KYB_FMT_COUNT || n <= 0 || k <= 0 || k % 256) return 0;
    return (size_t)((n + 15) / 16) * (size_t)(k / 256) * (size_t)kyb_tile_bytes(fmt);
}

size_t kyb_raw_row_bytes(int fmt, int64_t k) {
    if (fmt < 0 || fmt >= KYB_FMT_COUNT || k <= 0 || k % kyb_raw_block_elems(fmt)) return 0;
    return (size_t)(k / kyb_raw_block_elems(fmt)) * (size_t)kyb_raw_block_bytes(fmt);
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------ self-test of the bounded-wait report path
// One thread waits on an mbarrier that nothing ever completes, with the same bounded wait the kernels use and a small poll limit; when the wait gives up the
// kernel records a status code and returns by itself (no trap, no fault, nothing left in flight), exactly as a kernel whose copy never arrived would.
namespace kyb {
__global__ void selftest_wait_kernel(unsigned int* status, uint32_t polls) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
        if (!mbar_wait_bounded(&bar, 0, polls)) atomicExch(status, KYB_DEV_TIMEOUT_SELFTEST);
    }
}
}  // namespace kyb

extern "C" int kyb_selftest_wait_timeout(int polls, void* stream) {
    KYB_REQUIRE(polls >= 1 && polls <= 4096, "polls=%d: 1..4096", polls);
    unsigned int* w = kyb_device_status_word();
    KYB_REQUIRE(w, "could not set up the device status word");
    kyb::selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(w, (uint32_t)polls);
    return kyb_launch_check("selftest_wait");
}

// ------------------------------------------------------------------------------------------------ results of a step gathered into one buffer
// Up to 128 device arrays copied into one contiguous buffer by a single launch (16-byte units; sizes and addresses multiples of 16): the results of a decode step
// leave the device with one copy instead of one per product.
namespace kyb {
struct GatherList {
    const uint4* src[128];
    uint4* dst[128];
    uint32_t units[128];
    int count;
};
__global__ void gather_flat_kernel(const GatherList g) {
    const int j = blockIdx.y;
    if (j >= g.count) return;
    const uint4* s = g.src[j];
    uint4* d = g.dst[j];
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < g.units[j]; i += gridDim.x * blockDim.x) d[i] = s[i];
}
}  // namespace kyb

extern "C" int kyb_gather_flat(const void* const* srcs, void* const* dsts, const int64_t* bytes, int count, void* stream) {
    KYB_REQUIRE(srcs && dsts && bytes && count >= 1 && count <= 128, "1..128 arrays");
    kyb::GatherList g;
    uint32_t most = 0;
    for (int i = 0; i < count; ++i) {
        KYB_REQUIRE(srcs[i] && dsts[i] && bytes[i] > 0 && bytes[i] % 16 == 0 && bytes[i] < (1ll << 35), "array %d: null, empty or not a multiple of 16 bytes", i);
        KYB_REQUIRE(((uintptr_t)srcs[i] & 15) == 0 && ((uintptr_t)dsts[i] & 15) == 0, "array %d is not 16-byte aligned", i);
        g.src[i] = (const uint4*)srcs[i], g.dst[i] = (uint4*)dsts[i], g.units[i] = (uint32_t)(bytes[i] / 16);
        most = g.units[i] > most ? g.units[i] : most;
    }
    g.count = count;
    const unsigned bx = (unsigned)((most + 255) / 256 < 64 ? (most + 255) / 256 : 64);
    kyb::gather_flat_kernel<<<dim3(bx ? bx : 1, (unsigned)count), 256, 0, (cudaStream_t)stream>>>(g);
    return kyb_launch_check("gather_flat");
}
