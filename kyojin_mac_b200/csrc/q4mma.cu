// Few-row product on affine 4-bit weights (MLX layout): w uint32 [n, k/8] (element t of a word = nibble t), scales / biases fp16 [n, k/g], g = 32 or 64,
// weight = scale * q + bias. y[r, n] = sum_k x[r, k] * weight[n, k] for r < rows <= 32, fp32 accumulation, fp16 saturated output.
// Replaces the kernels of kyojin_mlx/q4mma.py:16-72, :110-187, :291-448 (`q4mma`, `q4mma3`, `q4mma4`). Q4_K reaches this entry through the affine view
// of its blocks (group 32, scale = fp16(d sc), bias = fp16(-dmin mn): kyojin_mlx/foreign_pack.py:136-176 `mq_arrays`), a tolerance-class path; the
// bit-exact, bandwidth-tuned path for Q4_K is kyb_gemv_t16.
// One pass over the weights for all rows, on the tensor cores: a warp owns 16 weight rows; per 32 inputs every lane loads ONE stored word of rows g and g + 8,
// four shift-and-mask steps turn its eight nibbles into the A operands of two mma.sync.m16n8k16 (codes as fp16 subnormals code * 2^-24, exact), the activations
// of up to 32 rows are the B operands (staged per 256 inputs in shared memory, one 16-byte load per lane and column tile, the k slots of a lane permuted to
// match the nibble order), and two more MMAs against a constant-one operand give the sums of x that the group's bias multiplies. Scale and bias are applied in
// fp32 to the 32-input partial sums. The result of an activation row does not depend on how many rows ride along.
#include "kyb_common.cuh"

namespace kyb {

constexpr int Q4_XPITCH = 288;      // halves per staged activation row: 256 + 32, so that rows g and g + 1 sit 64 bytes apart modulo 128 (conflict-free 16-byte loads)

template <int NT>
__global__ void __launch_bounds__(128) q4mma_kernel(const uint32_t* __restrict__ w, const __half* __restrict__ scales, const __half* __restrict__ biases, int group,
                                                    const __half* __restrict__ x, int64_t ldx, int rows, int n, int k, __half* __restrict__ y, int64_t ldy) {
    __shared__ __align__(16) __half xs[NT * 8][Q4_XPITCH];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int row0 = (blockIdx.x * 4 + warp) * 16;                              // this warp's 16 weight rows
    const int rg = min(row0 + g, n - 1), rh = min(row0 + g + 8, n - 1);         // rows past n repeat the last row; their results are not stored
    const uint32_t* wg = w + (size_t)rg * (k >> 3);
    const uint32_t* wh = w + (size_t)rh * (k >> 3);
    const int ng = k / group;
    const __half *sgp = scales + (size_t)rg * ng, *shp = scales + (size_t)rh * ng, *bgp = biases + (size_t)rg * ng, *bhp = biases + (size_t)rh * ng;
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    constexpr uint32_t ONE2 = 0x3C003C00u, M = 0x000F000Fu;                      // fp16 (1, 1); one nibble per 16-bit half
    for (int k0 = 0; k0 < k; k0 += 256) {
        __syncthreads();                                                          // the previous chunk has been consumed
        for (int idx = threadIdx.x; idx < NT * 8 * 32; idx += 128) {
            const int r = idx >> 5, q = idx & 31;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (r < rows && k0 + q * 8 < k) v = __ldg(reinterpret_cast<const uint4*>(x + (size_t)r * ldx + k0 + q * 8));
            *reinterpret_cast<uint4*>(&xs[r][q * 8]) = v;
        }
        __syncthreads();
        if (row0 >= n) continue;
#pragma unroll 2
        for (int c = 0; c < 8; ++c) {
            const int kk = k0 + 32 * c;
            if (kk >= k) break;
            const uint32_t a = __ldg(wg + (kk >> 3) + t), b = __ldg(wh + (kk >> 3) + t);    // elements kk + 8t .. + 7 of rows g, g + 8
            const int grp = kk / group;
            const float s_g = __half2float(sgp[grp]) * 16777216.0f, s_h = __half2float(shp[grp]) * 16777216.0f;     // the codes carry 2^-24
            const float b_g = __half2float(bgp[grp]), b_h = __half2float(bhp[grp]);
            // register j holds nibbles j and j + 4: elements (8t + j, 8t + j + 4)
            const uint32_t a0 = a & M, a1 = (a >> 4) & M, a2 = (a >> 8) & M, a3 = (a >> 12) & M;
            const uint32_t b0 = b & M, b1 = (b >> 4) & M, b2 = (b >> 8) & M, b3 = (b >> 12) & M;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint4 xv = *reinterpret_cast<const uint4*>(&xs[nt * 8 + g][32 * c + 8 * t]);    // x[row nt * 8 + g][kk + 8t .. + 7]
                const uint32_t x04 = prmt(xv.x, xv.z, 0x5410u), x15 = prmt(xv.x, xv.z, 0x7632u), x26 = prmt(xv.y, xv.w, 0x5410u), x37 = prmt(xv.y, xv.w, 0x7632u);
                float cq[4], cs[4];
                mma16816_z(cq, a0, b0, a1, b1, x04, x15);
                mma16816(cq, a2, b2, a3, b3, x26, x37);
                mma16816_z(cs, ONE2, ONE2, ONE2, ONE2, x04, x15);                   // every row: the sum of the 32 activations of each column
                mma16816(cs, ONE2, ONE2, ONE2, ONE2, x26, x37);
                acc[nt][0] = fmaf(s_g, cq[0], fmaf(b_g, cs[0], acc[nt][0]));
                acc[nt][1] = fmaf(s_g, cq[1], fmaf(b_g, cs[1], acc[nt][1]));
                acc[nt][2] = fmaf(s_h, cq[2], fmaf(b_h, cs[2], acc[nt][2]));
                acc[nt][3] = fmaf(s_h, cq[3], fmaf(b_h, cs[3], acc[nt][3]));
            }
        }
    }
    if (row0 >= n) return;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int m = nt * 8 + 2 * t + (q & 1), nrow = row0 + g + 8 * (q >> 1);
            if (m < rows && nrow < n) y[(size_t)m * ldy + nrow] = sat_half(acc[nt][q]);
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
    KYB_REQUIRE(n < (1ll << 31) && k < (1ll << 31), "dimension too large");
    const unsigned blocks = (unsigned)((n + 63) / 64);                           // four warps of 16 weight rows
    cudaStream_t st = (cudaStream_t)stream;
#define KYB_Q4(NT) kyb::q4mma_kernel<NT><<<blocks, 128, 0, st>>>((const uint32_t*)w, (const __half*)scales, (const __half*)biases, group, (const __half*)x, ldx, (int)rows, (int)n, (int)k, (__half*)y, ldy)
    if (rows <= 8) KYB_Q4(1);
    else if (rows <= 16) KYB_Q4(2);
    else KYB_Q4(4);
#undef KYB_Q4
    return kyb_launch_check("q4mma");
}
