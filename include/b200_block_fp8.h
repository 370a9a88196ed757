/*
 * C ABI of libb200_block_fp8.so -- the W8A8 block-FP8 linear path for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers, sizes and element strides; none
 * allocates, synchronises or reads device data on the host unless stated.  Kernels are
 * enqueued on `stream` (a cudaStream_t passed as void*; NULL = legacy default stream) of
 * the CURRENT device.  Return value: 0 on success, a negative B200_ERR_* code otherwise
 * (nothing is launched when an argument check fails); b200_strerror() names it.
 *
 * Each declaration cites the interface of the reference project (walker-ai/sglang,
 * paths relative to its checkout) that it stands in for.
 */
#ifndef B200_BLOCK_FP8_H_
#define B200_BLOCK_FP8_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of activations / outputs */
#define B200_DT_F32 0
#define B200_DT_F16 1
#define B200_DT_BF16 2

/* error codes */
#define B200_OK 0
#define B200_ERR_NULL_PTR (-1)
#define B200_ERR_BAD_DTYPE (-2)
#define B200_ERR_BAD_SHAPE (-3)      /* negative size, K % group != 0, ... */
#define B200_ERR_BAD_STRIDE (-4)     /* stride not allowed by the layout contract */
#define B200_ERR_MISALIGNED (-5)     /* pointer or leading dimension not 16-byte aligned */
#define B200_ERR_UNSUPPORTED (-6)    /* valid in the reference, not built here (see message) */
#define B200_ERR_CUDA (-7)           /* a CUDA runtime/driver call failed; see b200_last_cuda_error() */
#define B200_ERR_NOT_SM100 (-8)      /* current device is not compute capability 10.x */
#define B200_ERR_TOO_LARGE (-9)      /* size beyond a stated maximum */
#define B200_ERR_DEVICE_TIMEOUT (-10) /* a bounded device-side wait gave up (status word set) */

const char* b200_strerror(int code);
/* cudaError_t of the last failing CUDA call made by this library on this thread (0 if none). */
int b200_last_cuda_error(void);
/* Library ABI version (bumped on any signature change). */
int b200_abi_version(void);

/*
 * Per-token-group FP8 quantisation (e4m3, saturating, round-to-nearest-even).
 * Replaces: sgl_per_token_group_quant_fp8
 *   (sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:116-240, schema
 *    sgl-kernel/csrc/common_extension.cc:116-119).
 * x   [M,K] contiguous, x_dtype one of B200_DT_*; K % group_size == 0; group_size in {64,128,256,512}
 * q   [M,K] contiguous e4m3 codes (1 byte each)
 * s   fp32 scales; element (row r, group g) is written at s[r*s_stride_row + g*s_stride_grp].
 *     Row-major [M,G]: (G,1).  Column-major [G,M]: (1,M).  Column-major padded to 4 rows
 *     (TMA-aligned): (1, align4(M)); padding rows are not written.
 * Arithmetic (bit-exact with the reference kernel): amax = max(eps, max|float(x)|);
 * scale = amax / fp8_max (IEEE); code = e4m3_rne_sat(min(max(float(x)/scale, fp8_min), fp8_max)).
 * M == 0 is a no-op.
 */
int b200_per_token_group_quant_fp8(const void* x, int x_dtype, void* q, float* s,
                                   int64_t M, int64_t K, int64_t group_size,
                                   int64_t s_stride_row, int64_t s_stride_grp,
                                   float eps, float fp8_min, float fp8_max, void* stream);

/*
 * Per-token-group INT8 quantisation: the same operator with an int8 destination.
 * Replaces: sgl_per_token_group_quant_int8 (sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:219-228; the
 *   DST_DTYPE = int8_t launch at :206-207), called by sglang_per_token_group_quant_int8
 *   (python/sglang/srt/layers/quantization/int8_kernel.py:185-209).
 * Same layout arguments as above; q holds int8 codes.
 * Arithmetic (bit-exact with the reference kernel): amax = max(eps, max|float(x)|); scale = amax / int8_max (IEEE);
 * code = (int8) trunc(min(max(float(x)/scale, int8_min), int8_max)).
 */
int b200_per_token_group_quant_int8(const void* x, int x_dtype, void* q, float* s,
                                    int64_t M, int64_t K, int64_t group_size,
                                    int64_t s_stride_row, int64_t s_stride_grp,
                                    float eps, float int8_min, float int8_max, void* stream);

/* Same contract; divides with the IEEE division instruction sequence per element instead of
 * the reciprocal + exact-residual form.  Used by the tests to cross-check the fast form.
 * No counterpart in the reference. */
int b200_per_token_group_quant_fp8_ieee_div(const void* x, int x_dtype, void* q, float* s,
                                            int64_t M, int64_t K, int64_t group_size,
                                            int64_t s_stride_row, int64_t s_stride_grp,
                                            float eps, float fp8_min, float fp8_max, void* stream);

/*
 * Per-token-group (128) quantisation with power-of-two scales packed as biased-exponent bytes
 * (UE8M0), the scale_ue8m0 = true form of sgl_per_token_group_quant_fp8
 * (sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:54-61,86-97):
 *   s = exp2f(ceilf(log2f(max(amax / fp8_max, 1e-10f)))),  q = e4m3(clamp(x / s)),
 *   byte = (uint8)((int)log2f(s) + 127)
 * s_packed: int32 words holding four consecutive k-groups of one row (little-endian byte order), element
 * (row r, word w) at s_packed[w * s_stride_pack + r]  (s_stride_pack >= M; the reference passes
 * align4(M)).  Whole words are written: groups past K/128 inside the last word are zero bytes.
 */
int b200_per_token_group_quant_fp8_ue8m0(const void* x, int x_dtype, void* q, uint32_t* s_packed,
                                         int64_t M, int64_t K, int64_t s_stride_pack,
                                         float eps, float fp8_min, float fp8_max, void* stream);

/*
 * SiLU(gate) * up followed by per-token-group (128) FP8 quantisation in one pass: x [M, 2K] holds
 * gate | up per row (bf16 / fp16); writes codes q [M, K] and scales as above.  The product is formed
 * in fp32 and rounded to x's type before quantisation, so the result is bit-identical to
 * b200_silu_and_mul followed by b200_per_token_group_quant_fp8 while skipping the [M, K] round trip.
 * Replaces the pair silu_and_mul + sglang_per_token_group_quant_fp8 at
 * python/sglang/srt/layers/moe/cutlass_moe.py:191-194 (the reference fuses the same pair only in its
 * Triton EP path, python/sglang/srt/layers/moe/ep_moe/kernels.py:317-460).
 */
int b200_silu_mul_per_token_group_quant_fp8(const void* x, int x_dtype, void* q, float* s, int64_t M, int64_t K,
                                            int64_t s_stride_row, int64_t s_stride_grp, float eps, float fp8_min,
                                            float fp8_max, void* stream);

/*
 * b200_per_token_group_quant_fp8_ue8m0 with caller-chosen word strides: word (r, w) at
 * s_packed[r * s_stride_row + w * s_stride_pack].  s_stride_pack = 1 keeps a token's words together (the scale row
 * an expert-parallel dispatch copies per token).
 */
int b200_per_token_group_quant_fp8_ue8m0_strided(const void* x, int x_dtype, void* q, uint32_t* s_packed, int64_t M,
                                                 int64_t K, int64_t s_stride_row, int64_t s_stride_pack, float eps,
                                                 float fp8_min, float fp8_max, void* stream);

/*
 * The same fusion with power-of-two scales in the packed layout of b200_per_token_group_quant_fp8_ue8m0: the input
 * of the second expert GEMM on the block-scaling path.  Bit-identical to b200_silu_and_mul followed by
 * b200_per_token_group_quant_fp8_ue8m0.  Replaces silu_and_mul + sglang_per_token_group_quant_fp8(scale_ue8m0=True)
 * at python/sglang/srt/layers/moe/ep_moe/layer.py:606-628.
 */
int b200_silu_mul_per_token_group_quant_fp8_ue8m0(const void* x, int x_dtype, void* q, uint32_t* s_packed, int64_t M,
                                                  int64_t K, int64_t s_stride_pack, float eps, float fp8_min,
                                                  float fp8_max, void* stream);

/*
 * RMSNorm fused with the per-token-group (128) FP8 quantisation of its output -- the producer-side fusion of the
 * linear's quant stage.  y = T((x * rsqrt(mean(x^2) + norm_eps)) * weight) in fp32, rounded to x's type T exactly
 * as a separate norm kernel stores it, then quantised like b200_per_token_group_quant_fp8: codes and scales equal the
 * two-kernel sequence bit for bit, the [M, K] activation makes one trip through HBM instead of three.
 * residual != NULL: x + residual (fp32) is normalised and written back to residual rounded to T (fused_add_rmsnorm).
 * y != NULL: the normalised row is also stored.  q == s == NULL: the norm alone (y required).
 * scale_ue8m0 != 0: s is the packed exponent tensor (s_stride_grp = stride between packed words >= M).
 * x, residual, y: [M, K] contiguous bf16 / fp16; weight [K]; K % 128 == 0, K <= 16384.
 * Replaces: RMSNorm.forward (python/sglang/srt/layers/layernorm.py:78-171; sgl_kernel.rmsnorm /
 * fused_add_rmsnorm, sgl-kernel/python/sgl_kernel/elementwise.py:9-82) followed by
 * sglang_per_token_group_quant_fp8 at the head of w8a8_block_fp8_linear
 * (python/sglang/srt/layers/quantization/fp8_utils.py:199-201).
 */
int b200_rmsnorm_per_token_group_quant_fp8(const void* x, int x_dtype, void* residual, const void* weight, float norm_eps,
                                           void* y, void* q, void* s, int64_t M, int64_t K, int64_t s_stride_row,
                                           int64_t s_stride_grp, int scale_ue8m0, float eps, float fp8_min,
                                           float fp8_max, void* stream);

/*
 * Per-token-group (128) quantisation with a row gather: row r of q / s = the quantisation of row src_rows[r] of
 * x [x_rows, K] (indices clamped into the rows of x).  Same bits as quantising x and gathering codes and scales
 * afterwards.  scale_ue8m0 == 0: fp32 scales, element (r, g) at s[r * s_stride_row + g * s_stride_grp];
 * != 0: s is the packed exponent tensor of b200_per_token_group_quant_fp8_ue8m0 with s_stride_grp the stride between
 * packed words (>= R) and s_stride_row ignored.
 * Replaces: sglang_per_token_group_quant_fp8 + shuffle_rows (codes) + shuffle_rows (scales) at
 * python/sglang/srt/layers/moe/cutlass_moe.py:141-150; the quantise-then-ep_scatter pair of the reference's DeepGEMM
 * expert path (python/sglang/srt/layers/moe/ep_moe/layer.py:575-590).
 */
int b200_gather_per_token_group_quant_fp8(const void* x, int x_dtype, int64_t x_rows, const int32_t* src_rows, void* q,
                                          void* s, int64_t R, int64_t K, int64_t s_stride_row, int64_t s_stride_grp,
                                          int scale_ue8m0, float eps, float fp8_min, float fp8_max, void* stream);

/*
 * Dense block-scaled FP8 GEMM:  out[m,n] = cast( sum_kb ( sum_{k in kb} a[m,k]*b[n,k] )
 *                                               * sa[m,kb] * sb[n/128,kb] ),  fp32 accumulation.
 * Replaces: fp8_blockwise_scaled_mm
 *   (sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu:345-423, schema common_extension.cc:111-114)
 *   and w8a8_block_fp8_matmul (python/sglang/srt/layers/quantization/fp8_kernel.py:849-966).
 * a    [M,K] e4m3, row-major, leading dimension lda (elements) -- lda % 16 == 0, 16-byte aligned
 * b    [N,K] e4m3, row-major (= the reference's column-major [K,N] mat_b), ldb % 16 == 0
 * sa   fp32, element (m,kb) at sa[m*sa_stride_m + kb*sa_stride_g]   (M-major: (1, M) or (1, align4(M)))
 * sb   fp32, element (nb,kb) at sb[nb*sb_stride_n + kb*sb_stride_g]
 * out  [M,N] out_dtype (B200_DT_BF16 or B200_DT_F16; B200_DT_F32 is accepted for accuracy checks),
 *      leading dimension ldo elements, 16-byte aligned rows
 * K need not be a multiple of 128 (the last k-block is zero-filled); N need not be a multiple of 128.
 * M == 0 is a no-op.
 */
int b200_fp8_blockwise_scaled_mm(const void* a, int64_t lda, const void* b, int64_t ldb,
                                 const float* sa, int64_t sa_stride_m, int64_t sa_stride_g,
                                 const float* sb, int64_t sb_stride_n, int64_t sb_stride_g,
                                 void* out, int64_t ldo, int out_dtype,
                                 int64_t M, int64_t N, int64_t K, void* stream);

/*
 * The same product for small M (M <= 512), with the k-blocks of each output tile divided among
 * `split_k` CTAs so that the weight matrix streams through every SM even when the output has only a
 * few tiles (decode-size batches of the DeepSeek-V3 down projection: 28 tiles on 148 SMs).  Each CTA
 * writes fp32 partial sums to workspace[split][M][N]; a second kernel adds them in split order and
 * converts, so results are deterministic.  The fp32 sum over k-blocks is grouped differently from the
 * unsplit kernel, so the two agree to rounding (same parity tolerance), not bit for bit.
 *   split_k  0 = chosen by the library (falls back to 1 when the workspace is missing or too small);
 *            1 = identical to b200_fp8_blockwise_scaled_mm; 2..64 = forced (needs N % 4 == 0,
 *            split_k <= ceil(K/128))
 *   workspace  device memory, 16-byte aligned, at least split_k * M * N * 4 bytes; never allocated here
 * With split_k = 0 and M > 128 the library may instead split only the LAST WAVE of output tiles: when
 * tiles mod SMs is at most half of the SMs (896 tiles on 148 SMs leave a seventh wave of 8 tiles),
 * those tiles' k-blocks are divided among the SMs, their fp32 partial tiles go to the workspace (compact:
 * tail tiles x splits x 128 x tile width x 4 bytes) and a small second kernel adds them in split order.
 * Same rounding remark as above; the other tiles are bit-identical to the unsplit kernel.
 * b200_fp8_blockwise_scaled_mm_splitk_plan reports the split the library would choose for a shape on
 * a GPU with `sm_count` SMs (<= 0: 148) and the workspace that needs; it touches no device.
 * No counterpart in the reference (its CUTLASS kernel has no split-K form; the Triton kernel at
 * python/sglang/srt/layers/quantization/fp8_kernel.py:849-966 covers small M with smaller tiles).
 */
int b200_fp8_blockwise_scaled_mm_splitk(const void* a, int64_t lda, const void* b, int64_t ldb,
                                        const float* sa, int64_t sa_stride_m, int64_t sa_stride_g,
                                        const float* sb, int64_t sb_stride_n, int64_t sb_stride_g,
                                        void* out, int64_t ldo, int out_dtype,
                                        int64_t M, int64_t N, int64_t K,
                                        int split_k, void* workspace, size_t workspace_bytes, void* stream);
int b200_fp8_blockwise_scaled_mm_splitk_plan(int64_t M, int64_t N, int64_t K, int sm_count,
                                             int* split_k, size_t* workspace_bytes);

/*
 * The same product with the ACTIVATION scales given as packed UE8M0 exponent bytes, i.e. what
 * b200_per_token_group_quant_fp8_ue8m0 writes: element (m, kb) is byte kb % 4 of the 32-bit word at
 * sa_packed[(kb / 4) * sa_stride_pack + m * sa_stride_m], worth 2^(byte - 127).  Weight scales stay fp32
 * (power-of-two values after the reference's requantisation, but any fp32 value is accepted).
 * Stands in for w8a8_block_fp8_matmul_deepgemm on the activations side
 * (python/sglang/srt/layers/quantization/fp8_kernel.py:849-867, called from
 * deepgemm_w8a8_block_fp8_linear_with_fallback, fp8_utils.py:215-258).  The scales are decoded and
 * applied in fp32 exactly like the fp32-scale kernel; no hardware block scaling is used.
 */
int b200_fp8_blockwise_scaled_mm_ue8m0(const void* a, int64_t lda, const void* b, int64_t ldb,
                                       const uint32_t* sa_packed, int64_t sa_stride_m, int64_t sa_stride_pack,
                                       const float* sb, int64_t sb_stride_n, int64_t sb_stride_g,
                                       void* out, int64_t ldo, int out_dtype,
                                       int64_t M, int64_t N, int64_t K, void* stream);

/*
 * The same product on the tensor core's own block-scaling path (tcgen05.mma kind::mxf8f6f4.block_scale): BOTH scale
 * sets must be powers of two -- sa_packed as above, and sb_pow2 fp32 values 2^e (only their exponent field is
 * used; a mantissa that is not zero is ignored, i.e. the scale is rounded down to a power of two).  All k-blocks
 * accumulate inside tensor memory, nothing is promoted in fp32 registers, so this entry runs at the plain FP8 MMA
 * rate.  Power-of-two scaling is exact: results equal b200_fp8_blockwise_scaled_mm_ue8m0's up to the order of the
 * fp32 additions.  K % 128 == 0.
 * Replaces: the reference's DeepGEMM linear with UE8M0 scales, its default on Blackwell
 * (python/sglang/srt/layers/quantization/fp8_utils.py:215-258; weights re-quantised to power-of-two scales by
 * requant_weight_ue8m0, fp8_utils.py:370-443; python/sglang/srt/layers/deep_gemm_wrapper/entrypoint.py:78-93).
 */
int b200_fp8_blockwise_scaled_mm_pow2(const void* a, int64_t lda, const void* b, int64_t ldb, const uint32_t* sa_packed,
                                      int64_t sa_stride_m, int64_t sa_stride_pack, const float* sb_pow2,
                                      int64_t sb_stride_n, int64_t sb_stride_g, void* out, int64_t ldo, int out_dtype,
                                      int64_t M, int64_t N, int64_t K, void* stream);

/*
 * Grouped form of the block-scaling product, driven by a device-resident problem table: problem i multiplies rows
 * [problem_offsets[i], problem_offsets[i] + problem_rows[i * problem_rows_stride]) of a [total_rows, K] with weight
 * slice e = problem_experts[i] (i itself when problem_experts is NULL; a slice outside [0, num_weight_experts)
 * skips the problem) of b [num_weight_experts * N, K]; weight scales sb_pow2[e * sb_stride_e + (n/128) * sb_stride_n +
 * kb * sb_stride_g] are fp32 powers of two.  Packed activation exponents: word (row, g4) at
 * sa_packed[g4 * sa_stride_pack + row * sa_stride_m] with `row` the global row of a (sa_stride_problem < 0), or at
 * sa_packed[i * sa_stride_problem + g4 * sa_stride_pack + (row - problem_offsets[i]) * sa_stride_m] (>= 0).
 * Rows outside every problem are neither computed nor written.  At most 2048 problems; N % 128 == 0, K % 128 == 0.
 * Offsets and counts are clamped into the row range on the device.  Covers, with nothing read on the host:
 *   - the MoE expert GEMMs over rows packed without padding (problem_offsets / problem_rows = expert_offsets /
 *     column 0 of problem_sizes as b200_moe_prepare writes them),
 *   - DeepGEMM's CONTIGUOUS layout (one problem per 128-row block, problem_experts[i] = m_indices[128 * i]),
 *   - DeepGEMM's MASKED layout (problem i = expert i, problem_offsets[i] = i * max_m, problem_rows = masked_m,
 *     sa_stride_problem = the expert stride of the packed scales).
 * Replaces: deep_gemm.m_grouped_fp8_gemm_nt_contiguous / fp8_m_grouped_gemm_nt_masked behind
 * python/sglang/srt/layers/quantization/deep_gemm_wrapper/entrypoint.py:39-75 (callers
 * python/sglang/srt/layers/moe/ep_moe/layer.py:246-253,302-309,603-637).
 */
int b200_fp8_blockwise_scaled_grouped_mm_pow2(
    const void* a, int64_t lda, int64_t total_rows, const void* b, int64_t ldb, const uint32_t* sa_packed,
    int64_t sa_stride_m, int64_t sa_stride_pack, int64_t sa_stride_problem, const float* sb_pow2, int64_t sb_stride_e,
    int64_t sb_stride_n, int64_t sb_stride_g, void* out, int64_t ldo, int out_dtype, const int32_t* problem_offsets,
    const int32_t* problem_rows, int64_t problem_rows_stride, const int32_t* problem_experts, int num_problems,
    int num_weight_experts, int64_t N, int64_t K, void* stream);

/*
 * Expert GEMM 1 of the block-scaling path with the activation and the NEXT GEMM's quantisation in its epilogue:
 *   codes, exponents = quantise_pow2( SiLU(x W_gate^T) * (x W_up^T) )     (128-wide groups, packed words)
 * b holds 2 * N rows per weight slice (gate rows first), N = intermediate size; problems as in
 * b200_fp8_blockwise_scaled_grouped_mm_pow2.  The accumulator is rounded to mid_dtype (bf16 / fp16) before the
 * activation and the product after it, as the unfused kernels store them: the result equals
 * b200_fp8_blockwise_scaled_grouped_mm_pow2 followed by b200_silu_mul_per_token_group_quant_fp8_ue8m0 bit for bit,
 * and the [rows, 2N] intermediate never reaches HBM.  out_q [total_rows, N] e4m3 (leading dimension ldq bytes);
 * out_s: word (row, w) at out_s[w * out_s_stride_pack + row] (pass zeroed memory: bytes of absent groups are not
 * written).  N % 128 == 0, K % 128 == 0.
 * Replaces: grouped GEMM + silu_and_mul + sglang_per_token_group_quant_fp8 at
 * python/sglang/srt/layers/moe/cutlass_moe.py:171-194 / ep_moe/layer.py:603-628 -- the "GEMM epilogue that emits
 * e4m3 and scales" form of the fusion.
 */
int b200_fp8_blockwise_scaled_grouped_mm_pow2_silu_quant(
    const void* a, int64_t lda, int64_t total_rows, const void* b, int64_t ldb, const uint32_t* sa_packed,
    int64_t sa_stride_m, int64_t sa_stride_pack, int64_t sa_stride_problem, const float* sb_pow2, int64_t sb_stride_e,
    int64_t sb_stride_n, int64_t sb_stride_g, void* out_q, int64_t ldq, uint32_t* out_s, int64_t out_s_stride_pack,
    int mid_dtype, const int32_t* problem_offsets, const int32_t* problem_rows, int64_t problem_rows_stride,
    const int32_t* problem_experts, int num_problems, int num_weight_experts, int64_t N, int64_t K, void* stream);

/*
 * Grouped (per-expert) block-scaled FP8 GEMM: for every expert e,
 *   out[off_e : off_e + m_e, :] = blockscaled( a[off_e : off_e + m_e, :], b[e] )   (same math as above)
 * with off_e = expert_offsets[e], m_e = problem_sizes[3*e] read ON THE DEVICE (no host sync).
 * Replaces: fp8_blockwise_scaled_grouped_mm
 *   (sgl-kernel/csrc/moe/fp8_blockwise_moe_kernel.cu:587-743, schema common_extension.cc:192-197) and its
 *   helper get_group_gemm_starts (sgl-kernel/csrc/moe/cutlass_moe_helper.cu:10-142).
 * a    [total_rows, K] e4m3 row-major (rows grouped by expert), lda % 16 == 0
 * b    [E, N, K] e4m3, each expert row-major with leading dimension ldb, experts N*ldb apart
 * sa   fp32, element (row, kb) at sa[row*sa_stride_m + kb*sa_stride_g]  (row-major [rows, K/128]: (K/128, 1))
 * sb   fp32, element (e, nb, kb) at sb[e*sb_stride_e + nb*sb_stride_n + kb*sb_stride_g]
 * out  [total_rows, N]; rows not covered by any expert are left untouched
 * num_experts <= 1024.
 */
int b200_fp8_blockwise_scaled_grouped_mm(const void* a, int64_t lda, const void* b, int64_t ldb,
                                         const float* sa, int64_t sa_stride_m, int64_t sa_stride_g,
                                         const float* sb, int64_t sb_stride_e, int64_t sb_stride_n,
                                         int64_t sb_stride_g, void* out, int64_t ldo, int out_dtype,
                                         const int32_t* expert_offsets, const int32_t* problem_sizes,
                                         int num_experts, int64_t total_rows, int64_t N, int64_t K, void* stream);

/*
 * Routing tables for the grouped GEMMs, from topk_ids [num_tokens, topk] (int32; ids outside
 * [0, num_experts) get no slot -- expert-parallel masking):
 *   problem_sizes1[e] = (count_e, 2n, k), problem_sizes2[e] = (count_e, k, n),
 *   expert_offsets[0..E] exclusive prefix of count_e, blockscale_offsets (optional, may be NULL)
 *   prefix of count_e rounded up to 128, input_permutation[slot] = token, output_permutation[flat] = slot.
 * Slots inside an expert follow ascending flat index (deterministic; the reference uses atomics).
 * Replaces: prepare_moe_input (sgl-kernel/csrc/moe/prepare_moe_input.cu:13-167, schema
 *   common_extension.cc:198-202).
 * scratch: device memory of at least b200_moe_prepare_scratch_bytes(num_tokens*topk, num_experts) bytes,
 *   overwritten by the call (the reference allocates its own atomic buffer per call).
 */
size_t b200_moe_prepare_scratch_bytes(int64_t num_ids, int num_experts);
int b200_moe_prepare(const int32_t* topk_ids, int64_t num_tokens, int topk, int num_experts, int n, int k,
                     int32_t* expert_offsets, int32_t* blockscale_offsets, int32_t* problem_sizes1,
                     int32_t* problem_sizes2, int32_t* input_permutation, int32_t* output_permutation,
                     void* scratch, size_t scratch_bytes, void* stream);

/*
 * moe_align_block_size: replaces the op `moe_align_block_size`
 * (sgl-kernel/csrc/moe/moe_align_kernel.cu:283-366; declared sgl-kernel/include/sgl_kernel_ops.h:226; called from
 * python/sglang/srt/layers/moe/fused_moe_triton/fused_moe.py:558-628).
 * topk_ids: `numel` expert ids (int32, or int64 when ids_are_int64), -1 = filtered out.  num_experts counts the
 * SLOTS as in the reference (real experts + 1; slot = id + 1).  Outputs, all int32:
 *   sorted_token_ids[sorted_capacity]  flat indices grouped by slot, each slot's run padded to a multiple of
 *                                      block_size; padding positions are written (`numel`) only when
 *                                      pad_sorted_token_ids != 0, else the caller pre-filled them
 *   expert_ids[expert_ids_capacity]    slot - 1 of every block_size run
 *   num_tokens_post_pad[1]             total padded length
 *   cumsum_buffer[num_experts + 1]     padded exclusive prefix per slot
 * Inside a slot the flat indices ascend (the reference's order there is unspecified).  Ids outside
 * [-1, num_experts - 2] are skipped.  scratch: b200_moe_align_block_size_scratch_bytes(numel, num_experts)
 * bytes of device memory (0 for numel <= 4096: one launch; else three launches).  num_experts <= 2048.
 */
size_t b200_moe_align_block_size_scratch_bytes(int64_t numel, int num_experts);
int b200_moe_align_block_size(const void* topk_ids, int ids_are_int64, int64_t numel, int num_experts, int block_size,
                              int32_t* sorted_token_ids, int64_t sorted_capacity, int32_t* expert_ids,
                              int64_t expert_ids_capacity, int32_t* num_tokens_post_pad, int32_t* cumsum_buffer,
                              int pad_sorted_token_ids, void* scratch, size_t scratch_bytes, void* stream);

/*
 * b200_moe_prepare without scratch from the caller and without any allocation.  No counterpart in the
 * reference (its prepare_moe_input allocates a buffer on every call).
 * For callers that cannot obtain device memory where the routing tables are built -- a server whose
 * memory pool already owns the whole GPU, or a latency-critical section in which allocator calls
 * (which may synchronise the device) are not permitted.  The chunk-count table lives in a 256 KiB array inside the library (held on
 * every GPU that loads it until the process exits).
 * Limit: ceil(num_tokens*topk / 2048) * num_experts <= 65536, else B200_ERR_TOO_LARGE and nothing runs.
 * The first call on a device looks up the array's device address (one runtime query, no launch);
 * make that first call before any stream capture begins.
 * All calls on a device share the one array: the result does not depend on what an earlier call left
 * in it, but two calls whose kernels can overlap on the GPU (different streams, no ordering between
 * them) race on it -- order them, or use b200_moe_prepare with separate scratch.
 * Same outputs as b200_moe_prepare.
 */
int b200_moe_prepare_noalloc(const int32_t* topk_ids, int64_t num_tokens, int topk, int num_experts, int n, int k,
                             int32_t* expert_offsets, int32_t* blockscale_offsets, int32_t* problem_sizes1,
                             int32_t* problem_sizes2, int32_t* input_permutation, int32_t* output_permutation,
                             void* stream);

/*
 * Row gather of PACKED power-of-two scales (the layout of b200_per_token_group_quant_fp8_ue8m0: word w of row r at
 * [w * stride_pack + r]): output word (w, r) = input word (w, dst2src_map[r]), indices clamped into the source rows.
 * The companion of b200_shuffle_rows for the scales of the block-scaling expert path (the reference scatters codes
 * and scales together in ep_scatter, python/sglang/srt/layers/moe/ep_moe/kernels.py).
 */
int b200_shuffle_packed_scales(const uint32_t* input, int64_t input_stride_pack, int64_t num_src_rows,
                               const int32_t* dst2src_map, uint32_t* output, int64_t output_stride_pack,
                               int64_t num_dst_rows, int words_per_row, void* stream);

/* output[d, :] = input[dst2src_map[d], :] for rows of row_bytes bytes (128-bit copies when rows and
 * bases are 16-byte aligned, narrower ones otherwise).
 * Replaces: shuffle_rows (sgl-kernel/csrc/moe/prepare_moe_input.cu:169-256, schema :204-205). */
int b200_shuffle_rows(const void* input, const int32_t* dst2src_map, void* output, int64_t num_dst_rows,
                      int64_t row_bytes, void* stream);

/* out[r, :d] = silu(x[r, :d]) * x[r, d:2d] (fp32 math, one rounding); dtype B200_DT_BF16 / B200_DT_F16, d % 8 == 0.
 * Replaces: silu_and_mul (sgl-kernel/csrc/elementwise/activation.cu), as used between the two grouped
 * GEMMs at python/sglang/srt/layers/moe/cutlass_moe.py:191-192. */
int b200_silu_and_mul(const void* x, void* out, int64_t rows, int64_t d, int dtype, void* stream);

/* output[i, :] = sum_j factors[i*topk+j] * input[permutation[i*topk+j], :], j ascending, fp32 accumulation,
 * one rounding; factors may be NULL (all ones); permutation entries < 0 are skipped.
 * Replaces: apply_shuffle_mul_sum (sgl-kernel/csrc/moe/prepare_moe_input.cu:258-392, schema :206-207). */
int b200_apply_shuffle_mul_sum(const void* input, void* output, const int32_t* permutation, const void* factors,
                               int64_t m, int64_t topk, int64_t row_len, int dtype, void* stream);

/*
 * DeepSeek-V3 gate: s = sigmoid(gating_output); choice = s + bias; a group's score is the sum of its two
 * largest choice values; the topk_group best groups stay; the topk largest choice values among their experts
 * are picked (ties to the lower index); topk_weights = s[picked] / sum(s[picked]).
 * Replaces: moe_fused_gate (sgl-kernel/csrc/moe/moe_fused_gate.cu:56-260, schema common_extension.cc:176-179)
 * = biased_grouped_topk_impl with renormalize (python/sglang/srt/layers/moe/topk.py:462-530), without fused
 * shared experts.  gating_output [num_tokens, num_experts] fp32, bias [num_experts] fp32;
 * num_expert_group <= 32 divides num_experts (<= 1024), at least two experts per group, topk <= 32.
 */
int b200_moe_fused_gate(const float* gating_output, int64_t row_stride, const float* bias, float* topk_weights,
                        int32_t* topk_ids, int64_t num_tokens, int num_experts, int num_expert_group,
                        int topk_group, int topk, void* stream);
/* The same gate with the reference's fused shared experts (moe_fused_gate.cu:60-71,225-252): of the topk output
 * slots per token the last num_fused_shared_experts carry ids num_experts, num_experts + 1, ... and the weight
 * 1 / routed_scaling_factor (the reference's (sum / routed_scaling_factor) / sum); the first
 * topk - num_fused_shared_experts slots are the routed choices, renormalised over themselves. */
int b200_moe_fused_gate_shared_experts(const float* gating_output, int64_t row_stride, const float* bias,
                                       float* topk_weights, int32_t* topk_ids, int64_t num_tokens, int num_experts,
                                       int num_expert_group, int topk_group, int topk, int num_fused_shared_experts,
                                       double routed_scaling_factor, void* stream);

/*
 * Router: weights = softmax(gating_output.float(), dim=-1), then the topk largest per token and their expert
 * ids (ties to the lower id); with renormalize != 0 the k weights are divided by their sum.
 * Replaces: topk_softmax (sgl-kernel/csrc/moe/moe_topk_softmax_kernels.cu:502-570, schema
 * common_extension.cc:172) -- the kernel behind fused_topk (python/sglang/srt/layers/moe/topk.py:337-363).
 * gating_output [num_tokens, num_experts] fp32 / fp16 / bf16, rows row_stride elements apart;
 * topk_weights [num_tokens, topk] fp32, topk_ids [num_tokens, topk] int32.  num_experts <= 1024, topk <= 32.
 */
int b200_topk_softmax(const void* gating_output, int dtype, int64_t row_stride, float* topk_weights,
                      int32_t* topk_ids, int64_t num_tokens, int num_experts, int topk, int renormalize,
                      void* stream);

/*
 * Upper bound on the SMs the persistent kernels of this library occupy (their grids are sized by the SM count), for
 * the calling process; 0 = all.  Returns the previous value.  A row-parallel linear that overlaps the all-reduce of
 * one row chunk with the GEMM of the next leaves a few SMs to the all-reduce kernel this way (the reference reaches
 * the same end with deep_gemm.set_num_sms, python/sglang/srt/layers/quantization/deep_gemm_wrapper/entrypoint.py:100-110).
 * The value is read when a kernel is launched (or captured into a graph).  One setting per process, not synchronised:
 * a caller that launches from several threads sets it once, or serialises the launches it brackets with it.
 */
int b200_set_sm_limit(int sms);

/*
 * Sum of bf16 / fp16 buffers across 2..8 GPUs of one NVSwitch domain, one process per GPU.
 * Replaces: the reference's custom all-reduce (sgl-kernel/csrc/allreduce/custom_all_reduce.cuh, one-shot
 * and two-shot kernels over IPC peer pointers; registered as `all_reduce` in
 * sgl-kernel/csrc/common_extension.cc) and the NCCL all-reduce that RowParallelLinear.forward calls
 * (python/sglang/srt/layers/linear.py:1294-1300).
 *
 * peer_buffers[r] / peer_signal_pads[r]: rank r's symmetric buffer and signal pad (zero-initialised,
 * at least 4 * b200_allreduce_flag_words(world_size) bytes) as mapped into THIS process, r < world_size.
 * multicast_buffer: the multicast address of the buffer (NVLink SHARP: the switch adds), or NULL to use
 * peer loads and stores.  The range [offset_bytes, offset_bytes + bytes) of the buffer is reduced:
 *   one_shot = 0: in place on every rank (rank r reduces slice r and writes it to all ranks);
 *                 bytes % (16 * world_size) == 0.
 *   one_shot = 1: into `out` (local memory, bytes long); bytes % 16 == 0.  For small buffers.
 * Every element is the fp32 sum over ranks rounded once: identical bits on all ranks, run to run.
 * The kernels of the ranks wait for one another at flag barriers (bounded, about ten seconds): every rank
 * must call with the same arguments, in the same order, and nothing else may use the flag words
 * [flag_base_words, + b200_allreduce_flag_words(world_size)) of the signal pads meanwhile.  *status
 * (device memory, zero before the first call) receives a non-zero code if a peer never arrived; the
 * result is then undefined but the kernel still ends.  num_blocks: 0 = default, at most
 * b200_allreduce_max_blocks().
 */
int b200_allreduce(void* const* peer_buffers, void* const* peer_signal_pads, void* multicast_buffer, void* out,
                   int* status, int64_t offset_bytes, int64_t bytes, int dtype, int rank, int world_size,
                   int one_shot, int num_blocks, int64_t flag_base_words, void* stream);
int b200_allreduce_flag_words(int world_size);
int b200_allreduce_max_blocks(void);

/*
 * Expert-parallel token exchange over NVLink (2..8 GPUs of one NVSwitch domain, one process per GPU).
 * Replaces: the DeepEP dispatch / combine the reference's expert-parallel MoE uses
 * (python/sglang/srt/layers/moe/token_dispatcher/deepep.py:314-480, dispatch of quantised rows :328-336;
 * python/sglang/srt/layers/moe/ep_moe/layer.py:427-489); experts are split contiguously over the ranks
 * (python/sglang/srt/layers/moe/fused_moe_triton/layer.py:165-185).
 *
 * Every rank owns one symmetric buffer of b200_ep_buffer_bytes(...) bytes, mapped into every process
 * (peer_buffers[r], r < world_size) and laid out by the five byte offsets that call returns: receive regions
 * for codes [world][capacity][hidden] (e4m3), scales [world][capacity][hidden/128] (fp32) and
 * (local expert id, source slot) pairs [world][capacity] (2 x int32), a count table [world] (int32), and the
 * return buffer [max_slots][hidden] of the output type.  Zero the buffer once before the first call.
 *
 * b200_ep_dispatch: for every (token, choice) slot f = token*topk + j with expert e = topk_ids[f] >= 0, the
 *   token's row (q [num_tokens, hidden] e4m3, s [num_tokens, hidden/128] fp32 row-major) is stored into
 *   rank e / experts_per_rank's receive region for this source, at the slot's position among this source's
 *   rows for that rank (stable in f), together with (e % experts_per_rank, f).  A token's scales are
 *   scale_words_per_row consecutive 32-bit words of s (0 = hidden/128 fp32 scales; a multiple of 4, at most
 *   hidden/128: e.g. the packed power-of-two exponents with the words of a token contiguous and padded to four
 *   words); the receive region then holds rows of that many words.  Rows beyond `capacity` for one
 *   destination are dropped and *status becomes 31.  The call ends with a flag barrier between the ranks
 *   (flag words [flag_base_words, + world_size) of the signal pads), so kernels enqueued after it on the same
 *   stream see every peer's rows.  scratch_pos [num_tokens*topk] int32, scratch_counts [8] int32,
 *   scratch_counter [1] uint32 (zero before the first call): device scratch of the caller.
 * b200_ep_received_expert_ids: ids_out [world*capacity] int32 = the local expert id of each received row in
 *   region order, -1 where no row arrived (what the grouped GEMM's routing tables take as "skip").
 * b200_ep_combine: rows [*, hidden] (dtype bf16 / fp16) holds the expert output of received row r at row
 *   row_of[r] (r itself when row_of is NULL); each is stored into its source rank's return buffer at the row's
 *   source slot; ends with a flag barrier (a different flag_base_words than the dispatch's).
 * The kernels of the ranks wait for one another (bounded, about ten seconds): every rank must make the same
 * calls in the same order; *status (device word, zero before the first call) receives 32 / 33 if a peer
 * never arrived.  Nothing on the host reads device data.
 */
int64_t b200_ep_buffer_bytes(int world_size, int capacity, int hidden, int max_slots, int out_elem_bytes,
                             int64_t* layout_offsets_5);
int b200_ep_dispatch(const void* q, const void* s, int scale_words_per_row, const int32_t* topk_ids, int64_t num_tokens,
                     int topk, int hidden, int experts_per_rank, void* const* peer_buffers,
                     void* const* peer_signal_pads, const int64_t* layout_offsets_5, int capacity, int rank,
                     int world_size, int64_t flag_base_words, int* status, int32_t* scratch_pos, int32_t* scratch_counts,
                     unsigned int* scratch_counter, void* stream);
int b200_ep_received_expert_ids(const void* local_buffer, const int64_t* layout_offsets_5, int capacity, int hidden,
                                int world_size, int32_t* ids_out, void* stream);
int b200_ep_combine(const void* rows, const int32_t* row_of, int dtype, int hidden, void* const* peer_buffers,
                    void* const* peer_signal_pads, const int64_t* layout_offsets_5, int capacity, int rank,
                    int world_size, int64_t flag_base_words, int* status, unsigned int* scratch_counter, void* stream);

/*
 * Device-side waits in the GEMM kernels are bounded (about a second of SM clocks).  A wait that gives up
 * makes its kernel drain and exit, and records a code that is STICKY for the device, like a CUDA error:
 *   - every later GEMM entry point on that device returns B200_ERR_DEVICE_TIMEOUT without launching
 *     (the code is mirrored into pinned host memory, so this test costs no synchronisation);
 *   - b200_gemm_poll_status reads that host mirror (no synchronisation; 0 = nothing reported so far);
 *   - b200_gemm_device_status synchronises the device, returns the code and CLEARS it, after which
 *     launches are accepted again.
 * The output of the launch that gave up is undefined.  Launches that were already queued behind it are
 * not affected by it: each launch watches its own slot of a ring of status words, so a stale code can
 * never make a healthy kernel abandon its waits.  The first GEMM call on a device allocates the pinned
 * mirror (4 bytes); make that call before any stream capture.  No reference counterpart.
 */
int b200_gemm_device_status(int* status_out);
int b200_gemm_poll_status(int* status_out);

/*
 * Test hook (process-wide; no reference counterpart): which GEMM kernel the dispatcher picks, so that the
 * tests reach every kernel on every shape.  0 automatic; 128 / 256: the 128-token-tile kernel with that
 * tile width; 3: the weight-streaming kernel with its token tile chosen from the shape, 3032 / 3064 /
 * 3128: that token tile; 4: never the weight-streaming kernel.
 */
int b200_debug_force_block_n(int block_n);

#ifdef __cplusplus
}
#endif
#endif /* B200_BLOCK_FP8_H_ */
