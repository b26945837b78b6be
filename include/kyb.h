/* kyb.h - C ABI of the B200 (sm_100a) dequant-fused quantized linear.
 *
 * This is the drop-in boundary for the quantized-linear / routed-expert path of kyojin-mac. The reference has no
 * FFI for this path: its operators are Python functions that hand Metal kernel text to MLX
 * (kyojin_mlx/kernels.py:40-44 `_kern` -> mx.fast.metal_kernel). Each entry point below names the reference
 * function(s) whose device work it replaces; the Python mirror of those functions lives in kyojin_mac_b200/.
 *
 * Conventions
 *   - every pointer is a caller-owned DEVICE pointer unless it is named host_*; nothing here allocates device
 *     memory (scratch is passed in; sizes come from the *_workspace_bytes functions);
 *   - `stream` is a cudaStream_t passed as void*; calls are asynchronous on it and re-entrant across streams;
 *   - weights W are [n out rows, k inputs], activations x are row-major fp16 [m, k] with row stride ldx (elements),
 *     y = x W^T is fp16 [m, n] (row stride ldy), accumulated in fp32 and saturated to +-65504 (never inf), as the
 *     reference kernels do (kyojin_mlx/foreign_metal.py:344, :1076);
 *   - return value: KYB_OK or a negative status; kyb_last_error() gives the message of the calling thread's last
 *     failure. Shape or alignment violations are reported, never silently fixed.
 */
#ifndef KYB_H
#define KYB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KYB_OK            0
#define KYB_EINVAL       -1   /* bad shape, alignment, format or null pointer */
#define KYB_ECUDA        -2   /* a CUDA runtime call failed (message in kyb_last_error) */
#define KYB_ETIMEOUT     -3   /* a bounded device-side wait expired (reported through the status word) */
#define KYB_EUNSUPPORTED -4   /* valid request outside what this build implements */
#define KYB_EWORKSPACE   -5   /* scratch buffer missing or too small */

/* weight formats (GGUF block types of kyojin_mlx/foreign_gguf.py:27-35 TYPES; NVFP4 also in the qs/meta pack form) */
#define KYB_FMT_Q4_K  0
#define KYB_FMT_Q6_K  1
#define KYB_FMT_Q3_K  2
#define KYB_FMT_NVFP4 3
#define KYB_FMT_Q5_K  4
#define KYB_FMT_Q8_0  5
#define KYB_FMT_Q2_K  6
#define KYB_FMT_IQ4_XS 7  /* 4-bit indices into the non-linear IQ4_NL grid, one 6-bit scale per 32 inputs; every format is served by every entry point */
#define KYB_FMT_COUNT 8

#define KYB_DT_F32 0
#define KYB_DT_F16 1
#define KYB_DT_BF16 2

int kyb_version(void);
const char* kyb_status_string(int status);
const char* kyb_last_error(void);

/* ---- T16 layout (load time). Replaces kyojin_mlx/foreign_gguf.py:634-789 `to_pack` (lossless repack of the stored
 * blocks into the order the kernels read) and kyojin_mlx/fp4tile.py:72-134 `to_tile` / `from_tile`.
 * raw: GGUF rows [n, k / block_elems * block_bytes]; t16: kyb_t16_nbytes bytes (n padded to 16 rows with zero blocks). */
size_t kyb_t16_nbytes(int fmt, int64_t n, int64_t k);
size_t kyb_raw_row_bytes(int fmt, int64_t k);
int kyb_repack_raw_to_t16(int fmt, const void* raw, int64_t n, int64_t k, void* t16, void* stream);
int kyb_repack_t16_to_raw(int fmt, const void* t16, int64_t n, int64_t k, void* raw, void* stream);

/* ---- dequantise a T16 matrix to row-major [n, k] (ld elements per row), fp32 (bit-equal to
 * kyojin_mlx/foreign_gguf.py:376-394 `dequant` / foreign_pack.py:179-215 `dequant`) or fp16 (= that fp32 value rounded
 * to nearest, saturated). Replaces kyojin_mlx/foreign_linear.py:1050-1065 `DevPack.dequant` (kernels
 * foreign_metal.py:291-312 `dequant_source`, :1130-1146 `dequantk_source`). gscale: NVFP4 per-tensor scale (1 otherwise),
 * applied as one fp32 multiply (foreign_pack.py:213). Rows [row0, row0 + nrows) only (row0 % 16 == 0). */
int kyb_dequant_t16(int fmt, const void* t16, int64_t n, int64_t k, int64_t row0, int64_t nrows, float gscale,
                    int out_dtype, void* out, int64_t ld, void* stream);

/* gathered rows: out[i] = decoded row rows[i] (int32 ids on the device, 0 <= id < n), nrows rows of k weights. Token-embedding lookup in the stored blocks:
 * kyojin_mlx/foreign_linear.py:1170-1199 `StoredEmbedding.__call__` (mx.take of the per-row arrays + dequant). */
int kyb_dequant_rows_t16(int fmt, const void* t16, int64_t n, int64_t k, const void* rows, int64_t nrows, float gscale, int out_dtype, void* out, int64_t ld,
                         void* stream);

/* ---- decode GEMV, m <= 32 activation rows. Replaces kyojin_mlx/foreign_linear.py:846-857 `DevPack._gemv` /
 * `_gemvk` (kernels foreign_metal.py:115-202 `gemv_source`, :1004-1099 `_gemvk_source`) and the few-row products
 * :1025-1048 `_fmma` / `_mma` / :859-863 `_mmak`. The result of an activation row does not depend on m.
 * workspace: kyb_gemv_workspace_bytes bytes (may be 0 -> workspace may be NULL); split-k partial sums live there.
 * flags: 0, or KYB_GEMV_CHAINED = launch with programmatic stream serialization: the kernel's CTAs become resident, set up and start prefetching the WEIGHTS
 *   while the preceding kernel of the stream still drains, and wait for that kernel's completion only before they touch x, y or the workspace. Consecutive
 *   chained GEMVs of a decode step overlap their launch and pipeline-fill time this way (2 - 3 us per product). Rule for the caller: the weights must not be
 *   written by the kernel that directly precedes a chained call on the stream (weights loaded earlier and settled are fine; the Python modules pass the flag
 *   only from the second call of a matrix on). */
#define KYB_GEMV_CHAINED 1
size_t kyb_gemv_workspace_bytes(int fmt, int64_t n, int64_t k, int64_t m);
int kyb_gemv_t16(int fmt, const void* t16, int64_t n, int64_t k, const void* x, int64_t m, int64_t ldx, float gscale,
                 void* y, int64_t ldy, void* workspace, size_t workspace_bytes, int flags, void* stream);

/* the same product on a gated input: the row fed to the product is fp16(silu(a[r]) * b[r]) (a, b fp16 [m, k] with one row stride ldx; fp32 arithmetic, saturated;
 * limit > 0 clamps as kyb_silu_mul), formed while the rows are staged. Replaces kyojin_mlx/foreign_linear.py:960-977 `DevPack.apply_glu` (the reference folds the
 * activation into the x staging of its down product the same way). Bit-identical to kyb_silu_mul followed by kyb_gemv_t16. */
int kyb_gemv_glu_t16(int fmt, const void* t16, int64_t n, int64_t k, const void* a, const void* b, float limit, int64_t m, int64_t ldx, float gscale,
                     void* y, int64_t ldy, void* workspace, size_t workspace_bytes, int flags, void* stream);

/* ---- prefill GEMM on tcgen05 (UMMA 128 x 256 x 16, kind::f16, fp32 accumulation in tensor memory), fp16 operands:
 * d [m, n] = sat_f16(gscale * a [m, k] b [n, k]^T), k % 64 == 0, lda / ldb / ldd in elements. Replaces the library matmul of the
 * reference's large-row path, kyojin_mlx/foreign_linear.py:710 and :737 (`x2 @ self.dequant().T`), which the reference takes for
 * more rows than its stored kernels serve (thresholds at foreign_linear.py:38-81); b is the fp16 output of kyb_dequant_t16. */
int kyb_gemm_f16_tn(const void* a, int64_t lda, const void* b, int64_t ldb, int64_t m, int64_t n, int64_t k, float gscale,
                    void* d, int64_t ldd, void* stream);
/* the same product with the fp32 accumulators written out unrounded: d float [m, n] (ldd in floats, 16-byte aligned) */
int kyb_gemm_f16_tn_f32(const void* a, int64_t lda, const void* b, int64_t ldb, int64_t m, int64_t n, int64_t k, float gscale, void* d, int64_t ldd, void* stream);

/* grouped form: rows of a sorted by expert, b = expert stack [experts * n, k] in fp16, tile list on the device (tb, off from kyb_moe_plan with mt = 128),
 * optional scatter of the output rows (row_map) and per-expert output scale (gs). Replaces kyojin_mlx/foreign_kqgmm.py:225-239 `gmm` (tile lookup
 * :23-30 `_TILE`, scatter epilogue `orow`) and the `mx.gather_mm` fallback foreign_linear.py:1389-1407 `_sorted_gmm`. n % 128 == 0. */
int kyb_gemm_f16_grouped(const void* a, int64_t lda, const void* b, int64_t ldb, int64_t s, int64_t n, int64_t k, int experts, const void* tb,
                         const void* off, const void* row_map, const void* gs, void* d, int64_t ldd, void* stream);

/* ---- GEMM + all-gather in one kernel (N-sharded linear, one process per GPU): the epilogue stores every output tile into the [m, ld] output matrix of EVERY rank
 * (plain 16-byte stores to peer-mapped addresses over NVLink, own rank included) at column col0 = first output column of this rank's shard, so the slices are
 * gathered while the tensor cores work on the next tiles. The caller provides the peer-mapped base pointers (e.g. CUDA IPC or symmetric-memory mappings) and
 * synchronises the ranks around the call (all ranks must have finished reading the previous contents before, all kernels must have completed after). No
 * counterpart in the reference (it runs on one device); this is the N-sharding of the benchmark's multi-GPU configurations. */
typedef struct kyb_peer_out {
    void* ptr[8];   /* base address of the output matrix on rank i, as mapped into this process */
    int count;      /* ranks, 1..8 */
} kyb_peer_out;
int kyb_gemm_kq_ag(int fmt, const void* t16, int64_t n, int64_t k, const void* a, int64_t lda, int64_t m, float gscale, const kyb_peer_out* out, int64_t ldd, int64_t col0,
                   int msub, void* stream);
int kyb_gemm_nvfp4_ag(const void* a_codes, const void* sfa, const void* b_codes, const void* sfb, int64_t m, int64_t n, int64_t k, float gscale, int out_dtype,
                      const kyb_peer_out* out, int64_t ldd, int64_t col0, void* stream);

/* ---- prefill GEMM with the dequantisation fused into the tensor-core operand producer: weights are read as T16 tiles and decoded into shared memory, the fp16
 * matrix never exists in HBM. d fp16 [m, n] = sat(gscale * a fp16 [m, k] x W^T). Same call sites as the two entries above
 * (kyojin_mlx/foreign_linear.py:710 / :737 dense, kyojin_mlx/foreign_kqgmm.py:225-239 `gmm` grouped). Weights are rounded to fp16 at the reference's own rounding
 * points for its few-row tensor kernels (block scale and min to fp16, one fp16 fma per weight: kyojin_mlx/foreign_metal.py:1357-1358, :1382-1383); NVFP4 weights
 * are exact in fp16. msub = 0: chosen by the library (CTA pairs, tcgen05 cta_group::2, for more than 128 rows and one destination); 1 or 2: the one-CTA
 * kernel with that many 128-row blocks of a per work item (same bits either way). The grouped form needs n % 256 == 0 and tb / off from
 * kyb_moe_plan with the same mt (128 or 256 rows of one expert per work item). */
int kyb_gemm_kq(int fmt, const void* t16, int64_t n, int64_t k, const void* a, int64_t lda, int64_t m, float gscale, void* d, int64_t ldd, int msub, void* stream);
/* split-k form of kyb_gemm_kq for products with fewer 256 x 256 output tiles than SMs (the reference has no counterpart: its fallback for these row counts is
 * dequantise + library matmul, kyojin_mlx/foreign_linear.py:710 / :737). The 256-input blocks are cut into `split` equal ranges, (tile, range) items fill the
 * SMs, every item leaves its fp32 accumulator in the workspace, a second kernel adds the ranges in k order, scales, saturates and stores d. Deterministic; differs
 * from kyb_gemm_kq by the fp32 summation order only. kyb_gemm_kq_split: the factor the library suggests for a shape (1: do not split; splits keep ranges of at
 * least 2048 inputs). kyb_gemm_kq_split_bytes: size of the 16-byte aligned workspace = split * (m rounded up to 256) * (n rounded up to 256) * 4. */
int kyb_gemm_kq_split(int fmt, int64_t n, int64_t k, int64_t m);
size_t kyb_gemm_kq_split_bytes(int64_t n, int64_t m, int split);
int kyb_gemm_kq_splitk(int fmt, const void* t16, int64_t n, int64_t k, const void* a, int64_t lda, int64_t m, float gscale, void* d, int64_t ldd, int split,
                       void* workspace, size_t workspace_bytes, void* stream);
int kyb_gemm_kq_grouped(int fmt, const void* t16, int64_t n, int64_t k, int experts, const void* a, int64_t lda, int64_t s, const void* tb, const void* off,
                        const void* row_map, const void* gs, void* d, int64_t ldd, int mt, void* stream);
/* gate and up of a routed SwiGLU layer as ONE grouped product with the gated activation in its epilogue: an item's 256 weight rows are 128 rows of the gate stack
 * and the same 128 rows of the up stack; h fp16 [s, n] (sorted order) = silu(a) * b of the two products rounded to fp16 (what two kyb_gemm_kq_grouped calls would
 * store), optional clamp `limit` as kyb_silu_mul. Replaces gmm, gmm, silu_perm of kyojin_mlx/foreign_kqgmm.py:293-314 `mlp`. n % 128 == 0, ldh % 8 == 0. */
int kyb_gemm_kq_grouped_glu(int fmt, const void* t16_gate, const void* t16_up, int64_t n, int64_t k, int experts, const void* a, int64_t lda, int64_t s, const void* tb,
                            const void* off, const void* gs_gate, const void* gs_up, float limit, void* h, int64_t ldh, int mt, void* stream);

/* ---- NVFP4 on the block-scaled tensor-core path.
 * kyb_nvfp4_quant_rows: activations (x_dtype 1 = fp16, 2 = bf16) [rows, k] -> packed e2m1 codes [rows, k/2] (two per byte, low nibble first) + one e4m3 scale per
 *   16 inputs, written plain [rows, k/16] (sf_plain) and / or in the tensor-core chunk layout (sf_swz, kyb_nvfp4_sf_bytes bytes). The rounding rule is
 *   kyojin_mlx/fp4pack.py:30-48 `pack(x, block=16, e4m3_scale=True)`. kyb_nvfp4_unpack_rows is fp4pack.py:51-63 `unpack` (out_dtype 0 f32 / 1 f16 / 2 bf16).
 * kyb_nvfp4_sf_swizzle: plain scale bytes <-> chunk layout (128 rows x 4 scales per 512-byte chunk), lossless except that the sign bit is dropped and the NaN
 *   code 0x7F becomes 0, which is how the reference decodes them (kyojin_mlx/foreign_pack.py:113-117). Role of kyojin_mlx/fp4tile.py:72-134 `to_tile` / `from_tile`.
 * kyb_gemm_nvfp4: d [m, n] (out_dtype 1 = fp16 saturated, 2 = bf16) = gscale * A B^T with A, B packed e2m1 + block scales, tcgen05.mma kind::mxf4nvf4
 *   (block 16, fp32 accumulation in tensor memory). k % 256 == 0, n % 256 == 0. The reference has no W4A4 product (its NVFP4 linear is W4A16,
 *   kyojin_mlx/foreign_metal.py:1487-1557); this is the benchmark's "activations quantised on the fly with the same block rule" configuration.
 * kyb_fp4_quant_block32 / kyb_fp4_unpack_block32: the other form of the same codec, kyojin_mlx/fp4pack.py:30-63 with block = 32 and e4m3_scale = False: one
 *   exponent byte per 32 values (scale 2^(byte - 127), byte = ceil(log2(amax / 6)) + 127 with the amax floor 6 * 2^-126), same e2m1 codes. */
size_t kyb_nvfp4_sf_bytes(int64_t rows, int64_t k);
int kyb_fp4_quant_block32(const void* x, int x_dtype, int64_t ldx, int64_t rows, int64_t k, void* codes, void* scale_bytes, void* stream);
int kyb_fp4_unpack_block32(const void* codes, const void* scale_bytes, int64_t rows, int64_t k, int out_dtype, void* out, int64_t ldo, void* stream);
int kyb_nvfp4_quant_rows(const void* x, int x_dtype, int64_t ldx, int64_t rows, int64_t k, void* codes, void* sf_plain, void* sf_swz, void* stream);
int kyb_nvfp4_unpack_rows(const void* codes, const void* sf_plain, int64_t rows, int64_t k, int out_dtype, void* out, int64_t ldo, void* stream);
int kyb_nvfp4_sf_swizzle(void* plain, int64_t rows, int64_t k, void* swz, int to_swizzled, void* stream);
int kyb_gemm_nvfp4(const void* a_codes, const void* sfa, const void* b_codes, const void* sfb, int64_t m, int64_t n, int64_t k, float gscale, int out_dtype,
                   void* d, int64_t ldd, void* stream);

/* router logits in fp32: lg[t, r] = sum_h gw[r, h] * x[t, h] (x fp32 / fp16 / bf16 [T, H], gw fp32 [E, H]); column E = the shared-expert gate row sgw (fp32 [H]) when
 * sgw is not null. Replaces kyojin_mlx/foreign_moe.py:122-130 `_logits` (kernels :36-75). lg: fp32 [T, ldl], ldl >= E + (sgw ? 1 : 0). */
int kyb_router_logits(const void* x, int x_dtype, int64_t ldx, const void* gw, const void* sgw, int64_t T, int E, int64_t H, void* lg, int64_t ldl, void* stream);
/* Router logits on the tensor cores, for many tokens (prefill): the fp32 gate is cut ONCE into three fp16 pieces per row (kyb_router_split: s w = hi + 2^-11 mid +
 * 2^-22 lo with a power-of-two s per row, all 24 bits of w kept), each call then runs one tcgen05 GEMM of the fp16 activations on the stacked pieces with fp32
 * accumulation (every product is exact) and one launch that recombines the three partial sums. Same contraction as kyb_router_logits
 * (kyojin_mlx/foreign_moe.py:122-130) with a different summation order: equal to the fp64 logits within 1e-5 relative. rpad = kyb_router_rpad(E, has_shared);
 * pieces fp16 [3 rpad, H]; inv_scale float [rpad]; work float [T, 3 rpad], 16-byte aligned; x fp16, H % 64 == 0. */
int64_t kyb_router_rpad(int E, int has_shared);
int kyb_router_split(const void* gw, const void* sgw, int E, int64_t H, void* pieces, void* inv_scale, void* stream);
int kyb_router_logits_tc(const void* x, int64_t ldx, const void* pieces, const void* inv_scale, int64_t T, int E, int has_shared, int64_t H, void* work, void* lg,
                         int64_t ldl, void* stream);


/* ---- routed experts (MoE). Expert stacks are E matrices of n rows concatenated along rows (kyojin_mlx/foreign_linear.py:504-527).
 *
 * kyb_moe_select: router softmax + top-k + renormalise (+ sigmoid of the shared-expert gate logit at column E), one warp per token.
 *   Replaces kyojin_mlx/foreign_moe.py:77-104 `_SELECT` (launched by `_select` :132-135). logits fp32 [T, ld]; inds u32 [T*K]; scs f32 [T*K]; sgs f32 [T] or NULL.
 * kyb_moe_plan: counting sort of P slots by expert. Replaces kyojin_mlx/foreign_kqgmm.py:169-196 `_CSORT` / `csort` (order, tb, off) and
 *   kyojin_mlx/moe_sort.py:18-78 `plan_device` (tok, ids_s, wts_s, inv, cum = off). Any output may be NULL. Order inside an expert's segment is unspecified
 *   (as in the reference: moe_sort.py:10-12). ids i32 [P]; rank u32 [E] or NULL; mt = rows per tile for tb.
 * kyb_gather_rows: out[r] = x[src[r] / div] (optionally with a column permutation). Replaces foreign_kqgmm.py:242-268 `_GATHER_ORD` / `gather_perm`.
 * kyb_silu_mul: h = fp16(silu(a) * b) in fp32, optional clamp `limit` (> 0) and output column permutation. Replaces foreign_kqgmm.py:249-290 `_SILU_PERM` /
 *   `silu_perm`, foreign_moe.py:106-110 `_SILU`, foreign_linear.py:1275-1319 `glu_rows`.
 * kyb_moe_combine: o[t] = sum_k y[t K + k] * scs[t K + k] (+ sgs[t] * shared[t]); fp16 saturated or fp32. Replaces foreign_moe.py:112-119 `_COMBINE`.
 * kyb_moe_groups + kyb_gemv_group_t16: gathered GEMV over routed slots with expert election: slot s = expert eids[s] applied to row xrows[s] (or s / xdiv)
 *   of x; slots of one expert are served 8 at a time so its bytes are read once per 8 slots. Replace kyojin_mlx/foreign_linear.py:1068-1095 `DevPack.gather`
 *   (kernels foreign_metal.py:115-202 / :1004-1099 with gather=True, :1487-1557 `gemv_g2_source`, fp4tile.py:166-256) and kyojin_mlx/moe_union.py:27-129.
 *   g_expert u32 [S], g_slots u32 [8 S], ngroups u32 [1] are scratch written by kyb_moe_groups (one election serves every projection of a layer).
 *   gs: per-expert fp32 output scale or NULL. The two fusions of the reference's decode path are arguments of the same launch:
 *   t16b (with gsb) = a second stack of the same shape on the same slots, results in rows [S, 2 S) of y (gate | up in one launch,
 *   kyojin_mlx/foreign_linear.py:1119-1154 `gather_pair`); x2 = gated input, the row fed to the product is fp16(silu(x row) * x2 row) formed while it is
 *   staged, clamp `limit` > 0 as kyb_silu_mul (foreign_linear.py:1156-1164 `gather_glu`, kernel foreign_metal.py:1107-1113). eids (optional, u32 [S]):
 *   rows of y whose slot id is outside [0, E) are set to zero (such slots are in no group).
 *   Ids outside [0, E) (the router's 0xFFFFFFFF for a token with NaN logits) are tolerated everywhere: kyb_moe_plan sorts such slots behind the last
 *   segment with weight 0, kyb_gather_rows returns zeros for a source row >= xrows, the grouped products write zeros to their rows. */
int kyb_moe_select(const void* logits, int64_t ld, int64_t T, int E, int K, int norm, int has_shared, void* inds, void* scs, void* sgs, void* stream);
int kyb_moe_plan(const void* ids, const void* wts, const void* rank, int E, int64_t P, int topk, int mt, void* order, void* inv, void* tok, void* ids_s,
                 void* wts_s, void* off, void* tb, void* stream);
int kyb_gather_rows(const void* x, int64_t ldx, int64_t xrows, const void* src, int div, const void* perm, int64_t R, int64_t k, void* out, int64_t ldo, void* stream);
int kyb_silu_mul(const void* a, const void* b, int64_t ld, int64_t rows, int64_t n, float limit, const void* perm, void* h, int64_t ldh, void* stream);
int kyb_moe_combine(const void* y, int64_t ldy, const void* scs, const void* sgs, const void* shared, int64_t lds, int64_t T, int K, int64_t H, int out_dtype,
                    void* o, int64_t ldo, void* stream);
int kyb_moe_groups(const void* eids, int64_t S, int E, void* g_expert, void* g_slots, void* ngroups, void* stream);
int kyb_gemv_group_t16(int fmt, const void* t16, const void* t16b, int64_t n, int64_t k, int E, const void* x, const void* x2, float limit, int64_t ldx,
                       const void* eids, const void* xrows, int xdiv, int64_t S, const void* gs, const void* gsb, void* y, int64_t ldy, const void* g_expert,
                       const void* g_slots, const void* ngroups, void* stream);

/* two-step form with the partial sums exposed. Replaces kyojin_mlx/mma_gemv.py:129-135 `partial_mma` (-> f32 [parts, rows, n]) and :141-149 `finalize_rows`.
 * partial: f32 [kyb_gemv_chunks(n, k)][m][n padded to 16]; finalize adds the parts in k order, scales, saturates to fp16. */
int kyb_gemv_chunks(int64_t n, int64_t k);
int kyb_gemv_partial_t16(int fmt, const void* t16, int64_t n, int64_t k, const void* x, int64_t m, int64_t ldx, void* partial, void* stream);
int kyb_gemv_finalize(const void* partial, int chunks, int64_t m, int64_t n, float gscale, void* y, int64_t ldy, void* stream);

/* few-row product on affine 4-bit weights in the MLX layout (w u32 [n, k/8], scales / biases fp16 [n, k/group], group 32 or 64, weight = scale q + bias),
 * rows <= 32. Replaces kyojin_mlx/q4mma.py:97-106 `q4mma`, :451-474 `q4mma3` / `q4mma4` (kernels :16-72, :291-448). */
int kyb_q4mma(const void* w, const void* scales, const void* biases, int group, const void* x, int64_t ldx, int64_t rows, int64_t n, int64_t k,
              void* y, int64_t ldy, void* stream);

/* up to 128 device arrays copied by a single launch; addresses and sizes are multiples of 16 bytes; destinations may be peer-mapped addresses of other GPUs. Used by
 * the host-side step (kyojin_mac_b200/host_graph.py: the results of a decode step leave the device with one copy) and by the decode all-gather of N-sharded
 * linears (kyojin_mac_b200/dist.py PeerGather: every rank stores its output slices into all ranks' buffers with one launch per step). No counterpart in the
 * reference (unified memory, one device). */
int kyb_gather_flat(const void* const* srcs, void* const* dsts, const int64_t* bytes, int count, void* stream);

/* ---- kyb_gemv_t16 for callers that must not allocate device memory. No counterpart in the reference (MLX owns all allocation there).
 * Meant for hosts that cannot call cudaMalloc when they need a GEMV: a server that gave all free HBM to its KV-cache pool at start-up, a decode loop that
 * cannot afford the device-wide synchronisation cudaMalloc / cudaFree imply, or a runtime whose plug-in rules forbid the callee to allocate.
 * Same arithmetic and results as kyb_gemv_t16; the chunk sums and the bounded-wait status word live in a fixed 16 MiB + 256 B array inside the
 * library image (held by every GPU that loads the library until the process exits) instead of a caller workspace. The call allocates nothing
 * (no cudaMalloc / cudaFree, no allocating library routine). Limits and rules:
 *   - shapes whose chunk sums exceed 16 MiB (kyb_gemv_workspace_bytes) are refused with KYB_EWORKSPACE (use kyb_gemv_t16 with your own workspace);
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device current); make that first call
 *     before any stream capture;
 *   - all calls on a device share the one array: two calls that overlap on the GPU (different streams) race on it - serialise them;
 *   - check != 0: the call also synchronises `stream`, reads the status word and returns KYB_ETIMEOUT if a bounded wait expired (the word is cleared);
 *     check == 0: purely asynchronous, a timeout stays recorded until a later call with check != 0. */
int kyb_gemv_t16_static(int fmt, const void* t16, int64_t n, int64_t k, const void* x, int64_t m, int64_t ldx, float gscale,
                        void* y, int64_t ldy, int check, void* stream);

/* launch plan the GEMV would use (diagnostics): out8 = {column tiles, how work is dealt (1: whole row tiles per warp, one launch; 0: runs of chunks per warp,
 * chunk sums through the workspace and a finalize launch; 2: whole row tiles per CTA, chunk sums added in shared memory, one launch), warps per CTA, k-blocks
 * per canonical chunk, k-blocks per part, k parts, dynamic shared memory bytes, CTAs}. */
int kyb_gemv_plan(int fmt, int64_t n, int64_t k, int64_t m, int* out8);

/* device status word of the calling thread's current device: nonzero after a bounded wait expired inside a kernel.
 * kyb_check_device_status synchronises `stream`, reads and clears it. */
int kyb_check_device_status(void* stream);

/* self-test of that report path (no counterpart in the reference): launches one thread that waits, with the kernels' own bounded wait and a limit of `polls`
 * polls (1..4096), on a barrier that nothing completes. The wait gives up after well under a second, the kernel records a status code and returns by itself;
 * the next kyb_check_device_status on the stream returns KYB_ETIMEOUT and clears the word. Nothing faults and nothing is left in flight. */
int kyb_selftest_wait_timeout(int polls, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KYB_H */
