// Few-row product on affine 4-bit weights (MLX layout): w uint32 [n, k/8] (element t of a word = nibble t), scales / biases fp16 [n, k/g], g = 32 or 64,
// weight = scale * q + bias. y[r, n] = sum_k x[r, k] * weight[n, k] for r < rows <= 32, fp32 accumulation, fp16 saturated output.
// Replaces the kernels of kyojin_mlx/q4mma.py:16-72, :110-187, :291-448 (`q4mma`, `q4mma3`, `q4mma4`). Q4_K reaches this entry through the affine view
// of its blocks (group 32, scale = fp16(d sc), bias = fp16(-dmin mn): kyojin_mlx/foreign_pack.py:136-176 `mq_arrays`), a tolerance-class path; the
// bit-exact, bandwidth-tuned path for Q4_K is kyb_gemv_t16. One warp per output row; the result of an activation row does not depend on how many rows ride along.
#include "kyb_common.cuh"

namespace kyb {

template <int RB>
__global__ void q4mma_kernel(const uint32_t* __restrict__ w, const __half* __restrict__ scales, const __half* __restrict__ biases, int g, const __half* __restrict__ x,
                             int64_t ldx, int rows, int n, int k, __half* __restrict__ y, int64_t ldy) {
    const int warp = (int)(((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
    if (warp >= n) return;
    const uint32_t* wr = w + (size_t)warp * (k >> 3);
    const __half* sr = scales + (size_t)warp * (k / g);
    const __half* br = biases + (size_t)warp * (k / g);
    for (int r0 = 0; r0 < rows; r0 += RB) {
        float acc[RB];
#pragma unroll
        for (int r = 0; r < RB; ++r) acc[r] = 0.f;
        for (int i = lane; i < (k >> 3); i += 32) {
            const uint32_t word = wr[i];
            const int grp = (i << 3) / g;
            const float s = __half2float(sr[grp]), b = __half2float(br[grp]);
            float q[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) q[j] = (float)((word >> (4 * j)) & 15u);
#pragma unroll
            for (int r = 0; r < RB; ++r) {
                if (r0 + r < rows) {
                    const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x + (size_t)(r0 + r) * ldx + (size_t)i * 8));
                    const __half2* xh = reinterpret_cast<const __half2*>(&xv);
                    float dot = 0.f, sx = 0.f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __half22float2(xh[j]);
                        dot = fmaf(q[2 * j], f.x, dot);
                        dot = fmaf(q[2 * j + 1], f.y, dot);
                        sx += f.x + f.y;
                    }
                    acc[r] = fmaf(s, dot, fmaf(b, sx, acc[r]));
                }
            }
        }
#pragma unroll
        for (int r = 0; r < RB; ++r) {
            float v = acc[r];
#pragma unroll
            for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && r0 + r < rows) y[(size_t)(r0 + r) * ldy + warp] = sat_half(v);
        }
    }
}

}  // namespace kyb

extern "C" int kyb_q4mma(const void* w, const void* scales, const void* biases, int group, const void* x, int64_t ldx, int64_t rows, int64_t n, int64_t k, void* y,
                         int64_t ldy, void* stream) {
    KYB_REQUIRE(w && scales && biases && x && y, "null pointer");
    KYB_REQUIRE(group == 32 || group == 64, "group size %d: 32 or 64", group);
    KYB_REQUIRE(rows >= 1 && rows <= 32, "rows=%lld: this product serves 1..32 rows", (long long)rows);
    KYB_REQUIRE(n > 0 && k > 0 && k % 64 == 0 && ldx >= k && ldx % 8 == 0 && ldy >= n, "n=%lld k=%lld: k must be a multiple of 64, ldx of 8", (long long)n, (long long)k);
    KYB_REQUIRE(((uintptr_t)x & 15) == 0, "x must be 16-byte aligned");
    const int threads = 256;
    const unsigned blocks = (unsigned)((n * 32 + threads - 1) / threads);
    kyb::q4mma_kernel<4><<<blocks, threads, 0, (cudaStream_t)stream>>>((const uint32_t*)w, (const __half*)scales, (const __half*)biases, group, (const __half*)x, ldx, (int)rows, (int)n,
                                                                      (int)k, (__half*)y, ldy);
    return kyb_launch_check("q4mma");
}
