/*
 * helion_b200 -- C ABI of the sm_100a quantized-inference operators.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*, 0 = the legacy default stream), launches asynchronously on
 * that stream, never synchronises and never throws.  Unless its comment says
 * otherwise an entry point allocates nothing.  The return value is HB200_OK or
 * a negative HB200_ERR_* code; hb200_error_string() names it.
 *
 * Data formats (shared by all NVFP4 entry points):
 *   - packed e2m1: two 4-bit codes per byte along K, low nibble = even k
 *     (examples/nvfp4_gemm.py:396-408, examples/nvfp4_gemv.py:548-556);
 *   - block scales: one float8_e4m3fn byte per 16 K-elements, stored flat in
 *     the SWIZZLE_32_4_4 layout for logical shape [rows, K/16], zero padded to
 *     round_up(rows,128) x round_up(K/16,4) (examples/nvfp4_gemv.py:68-101).
 *
 * The reference (pytorch/helion) has no native FFI: its operators are Python
 * callables that JIT-compile generated kernels.  Each declaration below cites
 * the Python entry point whose device work it replaces.
 */
#ifndef HELION_B200_H_
#define HELION_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HB200_OK 0
#define HB200_ERR_INVALID_ARGUMENT (-1) /* null pointer, bad size or alignment   */
#define HB200_ERR_UNSUPPORTED (-2)      /* valid request outside built variants  */
#define HB200_ERR_CUDA (-3)             /* a CUDA runtime/driver call failed     */
#define HB200_ERR_DEVICE_TIMEOUT (-4)   /* a bounded device-side wait ran out    */
#define HB200_ERR_WORKSPACE (-5)        /* caller workspace missing or too small */
#define HB200_ERR_SCRATCH_LIMIT (-6)    /* shape needs more than the library's built-in scratch */

#define HB200_ABI_VERSION 1

int hb200_abi_version(void);
const char* hb200_error_string(int code);

/* --------------------------------------------------------------- NVFP4 GEMV
 * out[m, n] = bf16(alpha * sum_g scale[n, g] * sum_{i<16} e2m1(W[n, 16g+i]) * x[m, 16g+i])
 *
 * Replaces nvfp4_gemv_bf16in (examples/nvfp4_gemv.py:432-476,
 * pretuned_kernels/nvfp4_gemv/nvfp4_gemv.py:205-222) for batch == 1 and is its
 * decode-batch extension for 1 < batch <= 32 (x row-major [batch, K], out
 * row-major [batch, N]).  K % 16 == 0.  Activations are converted to fp16
 * before the multiply, as the reference's kernels do, so |x| must stay within
 * fp16 range.
 */
int hb200_nvfp4_gemv_bf16in(const void* weight_packed, /* u8  [N, K/2]            */
                            const void* x_bf16,        /* bf16 [batch, K]          */
                            const void* weight_scale,  /* e4m3 swizzled [N, K/16]  */
                            void* out_bf16,            /* bf16 [batch, N]          */
                            int64_t n, int64_t k, int64_t batch, float alpha, void* stream);

/* The batched kernel's arithmetic (block scale folded into the fp16 weight,
 * fp32 accumulation inside warp-level MMAs) for any batch in 1..32, including
 * batch == 1; exported so the two GEMV formulations can be cross-checked.
 * Same arguments as hb200_nvfp4_gemv_bf16in. */
int hb200_nvfp4_gemv_bf16in_mma(const void* weight_packed, const void* x_bf16, const void* weight_scale,
                                void* out_bf16, int64_t n, int64_t k, int64_t batch, float alpha, void* stream);

/* Replaces nvfp4_gemv_fp4in (examples/nvfp4_gemv.py:479-525): the activation is
 * itself NVFP4 (packed codes [K/2] and swizzled e4m3 scales for logical
 * [1, K/16]); the block scale applied is weight_scale * x_scale. */
int hb200_nvfp4_gemv_fp4in(const void* weight_packed, const void* x_packed, const void* weight_scale,
                           const void* x_scale, void* out_bf16, int64_t n, int64_t k, float alpha,
                           void* stream);

/* ------------------------------------------------- fused FP8 quant producers
 * Replaces silu_and_mul_per_block_quant
 * (pretuned_kernels/silu_and_mul_per_block_quant/silu_and_mul_per_block_quant.py:31-122).
 * input bf16 [tokens, 2*inter] (gate first, then up), row stride in_stride
 * elements; out e4m3 (or int8 when out_is_int8) [tokens, inter] with row stride
 * out_stride bytes; scales fp32 [tokens, inter/group] contiguous;
 * group in {64, 128}; scale_ub: optional device fp32 scalar (may be null). */
int hb200_silu_and_mul_per_block_quant(void* out, const void* input, void* scales, int64_t tokens,
                                       int64_t inter, int64_t in_stride, int64_t out_stride, int group,
                                       const float* scale_ub, int out_is_int8, void* stream);
/* The same for an input of another float type, as the reference converts any to fp32 first
 * (silu_and_mul_per_block_quant.py:99-107): in_dtype 0 = bf16, 1 = fp16, 2 = fp32. */
int hb200_silu_and_mul_per_block_quant_typed(void* out, const void* input, void* scales, int64_t tokens,
                                             int64_t inter, int64_t in_stride, int64_t out_stride, int group,
                                             const float* scale_ub, int out_is_int8, int in_dtype, void* stream);

/* Replaces rms_norm_dynamic_per_token_quant
 * (pretuned_kernels/rms_norm_dynamic_per_token_quant/rms_norm_dynamic_per_token_quant.py:40-128).
 * input/weight/residual bf16 or fp16 (in_is_fp16); result e4m3 or int8
 * [tokens, hidden] contiguous; scale fp32 [tokens]; residual (nullable) is
 * added to the input first and overwritten with the sum. */
int hb200_rms_norm_dynamic_per_token_quant(void* result, const void* input, const void* weight, void* scale,
                                           int64_t tokens, int64_t hidden, float epsilon,
                                           const float* scale_ub, void* residual, int in_is_fp16,
                                           int out_is_int8, void* stream);

/* Replaces per_token_group_fp8_quant
 * (pretuned_kernels/per_token_group_fp8_quant/per_token_group_fp8_quant.py:29-74);
 * arithmetic follows the module's fp32 reference (:77-97).
 * input bf16/fp16/fp32 (in_dtype 0/1/2) [tokens, hidden] contiguous. */
int hb200_per_token_group_fp8_quant(const void* input, void* output_q, void* output_s, int64_t tokens,
                                    int64_t hidden, int group, float eps, float fp8_min, float fp8_max,
                                    int scale_ue8m0, int in_dtype, void* stream);

/* ------------------------------------------------------- NVFP4 quantiser
 * bf16 [rows, K] (row stride ldx elements) -> packed e2m1 codes [rows, K/2],
 * e4m3 block scales in SWIZZLE_32_4_4 order for logical [rows, K/16] (only the
 * logical entries are written: the caller zero-fills the buffer when rows % 128
 * or (K/16) % 4 is non-zero) and the fp32 global scale g = amax / (6*448):
 *   per_token == 0: *global_scale is an input, one value for the tensor;
 *   per_token != 0: global_scale[rows] is an output, one value per row.
 * Codes follow quantize_fp4_e2m1 (examples/nvfp4_gemm.py:368-381); the
 * reference has no kernel for this step (it calls vLLM's scaled_fp4_quant,
 * pretuned_kernels/nvfp4_gemv/nvfp4_gemv.py:241-246). */
int hb200_nvfp4_quantize(const void* x_bf16, void* codes, void* scales_swizzled, float* global_scale,
                         int64_t rows, int64_t k, int64_t ldx, int per_token, void* stream);

/* Per-token NVFP4 quantisation with fan-out, the dispatch step of the NVFP4 MoE layer in one pass: token t of
 * x [tokens, k] (bf16, row pitch ldx) is quantised once and its packed row, block scales and global scale are
 * written to the rows dst_rows[t * fanout .. (t + 1) * fanout) of the expert-sorted padded layout (negative
 * entries are skipped).  Same bytes as hb200_nvfp4_quantize + hb200_moe_gather_rows.  k % 64 == 0, k <= 4096,
 * fanout <= 32.  No counterpart in the reference (its MoE example gathers bf16 rows inside the GEMM,
 * examples/moe_matmul_ogs.py:58-66). */
int hb200_nvfp4_quantize_scatter(const void* x_bf16, void* codes, void* scales_swizzled, float* global_scale,
                                 const int32_t* dst_rows, int64_t tokens, int64_t fanout, int64_t k, int64_t ldx,
                                 void* stream);

/* RMSNorm fused with per-token NVFP4 quantisation (the NVFP4 form of rms_norm_dynamic_per_token_quant, whose
 * normalisation arithmetic it keeps: pretuned_kernels/rms_norm_dynamic_per_token_quant/
 * rms_norm_dynamic_per_token_quant.py:131-150): x [rows, k] bf16 (row pitch ldx), weight [k] bf16 -> codes
 * [rows, k/2], swizzled scales for [rows, k/16], global_scale[rows] = row_amax / (6 * 448).  The reference has no
 * NVFP4 producer (it leans on vLLM's scaled_fp4_quant, pretuned_kernels/nvfp4_gemv/nvfp4_gemv.py:241-246).
 * The SiLU-mul form of the same producer is hb200_nvfp4_quantize_rows with silu_mul = 1. */
int hb200_rms_norm_nvfp4_quant(const void* x_bf16, const void* weight_bf16, void* codes, void* scales_swizzled,
                               float* global_scale, int64_t rows, int64_t k, int64_t ldx, float epsilon,
                               void* stream);

/* ------------------------------------------------------------ NVFP4 GEMM
 * D[M, N] = out_dtype(alpha * A[M, K] . B[N, K]^T), both operands packed e2m1
 * and K-major, e4m3 block scales in SWIZZLE_32_4_4 order for logical [M, K/16]
 * and [N, K/16], fp32 accumulation on the tensor cores
 * (tcgen05.mma kind::mxf4nvf4).  Replaces nvfp4_scaled_matmul
 * (examples/nvfp4_gemm.py:331-364, which defers to torch._scaled_mm); alpha
 * carries the product of the operands' global scales (1.0 reproduces the
 * reference call).  out_dtype: 0 bf16, 1 fp16, 2 fp32; ldc in elements.
 * K % 32 == 0; all pointers 16-byte aligned. */
int hb200_nvfp4_scaled_matmul(const void* a_packed, const void* b_packed, const void* scale_a,
                              const void* scale_b, void* out, int64_t m, int64_t n, int64_t k, int64_t ldc,
                              float alpha, int out_dtype, void* stream);

/* ------------------------------------------------------- grouped NVFP4 GEMM
 * The MoE expert GEMM: out[r, :] = out_dtype(alpha * group_alpha[g] * row_scale[r]
 * * A[r, :] . B[g]^T) for every row r of group g.  Rows of A (and of out) are laid
 * out group after group, each group padded to a multiple of 128 rows, as produced
 * by hb200_moe_build_schedule; tile_info holds (group, valid rows) per 128-row
 * tile as int32 pairs, group < 0 for unused tiles (read on the device only).
 * b_packed is [groups, N, K/2]; scale_b holds one swizzled [N, K/16] buffer per
 * group, back to back; scale_a is the swizzled buffer for logical
 * [max_m_tiles*128, K/16].  row_scale / group_alpha may be null.
 * Generalises grouped_gemm_deepgemm's worklist form
 * (pretuned_kernels/grouped_gemm_deepgemm/grouped_gemm_deepgemm.py:172-224) and
 * moe_matmul_ogs (examples/moe_matmul_ogs.py:31-85) to NVFP4 operands. */
int hb200_nvfp4_grouped_matmul(const void* a_packed, const void* b_packed, const void* scale_a,
                               const void* scale_b, void* out, const int32_t* tile_info, int64_t max_m_tiles,
                               int64_t n, int64_t k, int64_t groups, int64_t ldc, const float* row_scale,
                               const float* group_alpha, float alpha, int out_dtype, void* stream);

/* Device-side schedule of the grouped GEMM from a routing result (no host read):
 * counts[experts] tokens per expert and sorted_pairs[pairs] = the (token, slot)
 * pairs (token * top_k + slot) ordered by expert, stably.  Writes
 * padded_offsets[experts+1], tile_info[max_tiles] (int32 pairs), the padded row of
 * every sorted position and of every pair.  Replaces the host bookkeeping of
 * moe_matmul_ogs_helion_kernel_args_gen (examples/moe_matmul_ogs.py:89-124). */
int hb200_moe_build_schedule(const int32_t* counts, int64_t experts, const int32_t* sorted_pairs, int64_t pairs,
                             int32_t* padded_offsets, int32_t* tile_info, int64_t max_tiles,
                             int32_t* row_of_sorted, int32_t* row_of_pair, void* stream);

/* Per-token NVFP4 quantisation of gathered rows; with silu_mul != 0 the row is
 * bf16(silu(x[:, :k]) * x[:, k:2k]) of a [*, 2k] input.  Item i reads source row
 * src_idx[i] / src_div (i if src_idx is null) and writes at row dst_idx[i] (i if
 * null); global_scale[row] = row_amax / (6*448) * item_scale[i] (1 if null).
 * No reference counterpart (see hb200_nvfp4_quantize). */
int hb200_nvfp4_quantize_rows(const void* x_bf16, void* codes, void* scales_swizzled, float* global_scale,
                              int64_t items, int64_t k, int64_t ldx, const int32_t* src_idx, int src_div,
                              const int32_t* dst_idx, const float* item_scale, int silu_mul, void* stream);

/* Copies per-token NVFP4 rows (codes [*, K/2], swizzled scales, global scale) into the
 * expert-sorted padded layout: item i reads token src_pair[i] / src_div and writes row
 * dst_row[i] (scales are re-swizzled for the destination row).  K % 32 == 0.  No
 * reference counterpart. */
int hb200_moe_gather_rows(const void* codes_in, const void* scales_in, const float* g_in, void* codes_out,
                          void* scales_out, float* g_out, const int32_t* src_pair, int src_div,
                          const int32_t* dst_row, int64_t items, int64_t k, void* stream);

/* out[t, :] = bf16(sum_s w[t, s] * expert_out[row_of_pair[t * top_k + s], :]) in
 * fp32, slot order; w = pair_weight (fp32 [tokens * top_k]) or 1 when null.  No
 * reference counterpart (the reference has no top-k combine). */
int hb200_moe_combine(const void* expert_out_bf16, int64_t ld, const int32_t* row_of_pair,
                      const float* pair_weight, void* out_bf16, int64_t tokens, int64_t top_k, int64_t hidden,
                      void* stream);

/* ------------------------------------------------ bf16 / fp16 grouped GEMM
 * out[r, :] = A[r, :] . B[g]^T for the rows of every row tile, fp32 accumulate on
 * the tensor cores (tcgen05 kind::f16), output in the input dtype.  A [a_rows, K]
 * and B [groups * N, K] are K-major.  row_tiles holds int32 quadruples
 * (group, first row, valid rows, rows to store) of at most 128 rows each: rows
 * past "valid" are written as zero up to "store", rows past "store" are not
 * written, a negative group marks an unused entry (read on the device only).
 * Replaces the device work of grouped_gemm_deepgemm
 * (pretuned_kernels/grouped_gemm_deepgemm/grouped_gemm_deepgemm.py:172-224),
 * moe_matmul_ogs (examples/moe_matmul_ogs.py:31-85) and grouped_gemm_jagged
 * (examples/grouped_gemm.py:52-104).  K % 8 == 0. */
int hb200_grouped_gemm_f16(const void* a, const void* b, void* out, const int32_t* row_tiles,
                           int64_t num_row_tiles, int64_t a_rows, int64_t n, int64_t k, int64_t groups,
                           int64_t ldc, int is_bf16, void* stream);

/* Direct mode of the reference's grouped GEMM (pretuned_kernels/grouped_gemm/grouped_gemm.py:213-327): group i is an
 * NT GEMM of its own, out_i[m_i, n_i] = A_i[m_i, k_i] . B_i[n_i, k_i]^T (fp32 accumulate), with per-group N and K
 * and operands / outputs anywhere in device memory.  The reference hands its kernel device tables of pointers and
 * strides built from host values; this entry point takes those host values: every array argument is a HOST array
 * of `groups` entries, lda / ldb / ldc are row pitches in elements (unit stride along K and N).  Groups with
 * m, n or k == 0 are skipped (their outputs are left as they are).  k_i % 8 == 0, row pitches of A and B % 8 == 0,
 * operand bases 16-byte aligned (HB200_ERR_UNSUPPORTED otherwise).  One launch per eight groups. */
int hb200_grouped_gemm_f16_direct(const void* const* a_ptrs, const void* const* b_ptrs, void* const* out_ptrs,
                                  const int64_t* m, const int64_t* n, const int64_t* k, const int64_t* lda,
                                  const int64_t* ldb, const int64_t* ldc, int64_t groups, int is_bf16, void* stream);

/* Row tiles of a jagged layout from device-resident group offsets [groups + 1]
 * (no host read): one entry per 128 rows of every group, unused entries marked.
 * max_tiles >= total_rows / 128 + groups always suffices. */
int hb200_build_row_tiles(const int32_t* group_offsets, int64_t groups, int32_t* row_tiles, int64_t max_tiles,
                          void* stream);

/* Tile list from device-resident per-group row counts (the device split sizes of the reference's grouped
 * tcgen05 kernels, test/test_cute_grouped_gemm_split_sizes.py:620-745): group g owns rows [P_g, P_g + size_g),
 * P the raw running sum; a size is clipped to [0, total_rows] in 64 bits, the interval to [0, total_rows), so
 * oversized, negative and beyond-int32 sizes never reach outside the matrices.  sizes int64 or int32 with an
 * element stride; groups <= 1024. */
int hb200_build_split_tiles(const void* split_sizes, int sizes_are_i64, int64_t stride, int64_t groups,
                            int64_t total_rows, int32_t* row_tiles, int64_t max_tiles, void* stream);

/* Tile list for a worklist [items, 4] of (group, start row, valid rows, rows to store), the metadata
 * grouped_gemm_deepgemm takes (pretuned_kernels/grouped_gemm_deepgemm/grouped_gemm_deepgemm.py:172-224), built
 * on the device.  Items are not trusted: negative group or start drops the item, store is clipped to the rows
 * that exist, valid to store.  max_tiles >= ceil(total_rows / 128) + items suffices for non-overlapping items;
 * tiles past max_tiles are dropped.  items <= 8192. */
int hb200_build_worklist_tiles(const int32_t* worklist, int64_t items, int64_t total_rows, int32_t* row_tiles,
                               int64_t max_tiles, void* stream);

/* silu_mul_fp8 (pretuned_kernels/silu_mul_fp8/silu_mul_fp8.py:29-59): out[t, j] = fp8_e4m3(p * (1 / scale)) with
 * p = input_dtype(input_dtype(silu(x[t, j])) * x[t, d + j]), one static fp32 scale (device pointer), input
 * [tokens, 2 d] bf16 (in_is_fp16 = 0) or fp16 with row pitch in_stride elements, out [tokens, d] contiguous.
 * Values beyond the e4m3 range saturate to +-448.  d % 8 == 0 and in_stride % 8 == 0 (HB200_ERR_UNSUPPORTED
 * otherwise). */
int hb200_silu_mul_fp8(void* out, const void* input, const float* scale, int64_t tokens, int64_t d,
                       int64_t in_stride, int in_is_fp16, void* stream);

/* ------------------------------------------------ row-wise scaled FP8 GEMM
 * scaled_mm (pretuned_kernels/scaled_mm/scaled_mm.py:18-84):
 *   c[m, n] = out_dtype(scale_b[n] * (scale_a[m] * sum_k a[m, k] * b[k, n])) + bias[n]
 * on the tensor cores (tcgen05 kind::f8f6f4, fp32 accumulate).  a [M, K] with row pitch lda, b given as its
 * K-major storage [N, K] with row pitch ldb (the reference's b [K, N] with b.stride(0) == 1), c [M, N] with row
 * pitch ldc, pitches in elements.  scale_a / scale_b are fp32, one value or one per row of a / column of b
 * (scale_a_per_row / scale_b_per_col); bias is [N] in the output type or null and is added after the cast, as
 * the reference does.  fp8_format 0 = e4m3, 1 = e5m2, 2 = int8 (both operands; int8 runs kind::i8 with an int32
 * accumulator, converted to fp32 once after the whole K range, scaled_mm.py:53); out_dtype 0 bf16, 1 fp16, 2 fp32.
 * Needs 16-byte aligned a and b and lda % 16 == ldb % 16 == 0 (HB200_ERR_UNSUPPORTED otherwise).
 * The (tile, K block) units are dealt to the CTAs in equal contiguous ranges; tiles shared between CTAs are
 * summed in a fixed order through `workspace`: caller-owned device memory of
 * hb200_fp8_scaled_mm_workspace_bytes(m, n, k) bytes (0 when the ranges end on tile boundaries) whose first
 * 16 KB are zero before the first call and are left zero by every call; HB200_ERR_WORKSPACE if it is missing
 * or too small.  Calls that share a workspace must not overlap. */
int64_t hb200_fp8_scaled_mm_workspace_bytes(int64_t m, int64_t n, int64_t k);
int hb200_fp8_scaled_mm(const void* a, const void* b, void* c, const float* scale_a, const float* scale_b,
                        const void* bias, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                        int scale_a_per_row, int scale_b_per_col, int fp8_format, int out_dtype, void* workspace,
                        int64_t workspace_bytes, void* stream);

/* rms_norm_per_block_quant (pretuned_kernels/rms_norm_per_block_quant/rms_norm_per_block_quant.py:38-140):
 * the RMSNorm of hb200_rms_norm_dynamic_per_token_quant with one scale per group of 64 or 128 elements of the
 * hidden dimension (true division for fp8, reciprocal multiply and round for int8).  Scale (t, g) is written at
 * scale[t * scale_stride_t + g * scale_stride_g] (fp32 elements), which covers the transposed scale layout. */
int hb200_rms_norm_per_block_quant(void* result, const void* input, const void* weight, void* scale, int64_t tokens,
                                   int64_t hidden, float epsilon, const float* scale_ub, void* residual,
                                   int group_size, int64_t scale_stride_t, int64_t scale_stride_g, int in_is_fp16,
                                   int out_is_int8, void* stream);

/* dynamic_per_token_scaled_fp8_quant
 * (pretuned_kernels/dynamic_per_token_scaled_fp8_quant/dynamic_per_token_scaled_fp8_quant.py:32-72):
 * scale[t] = max(min(amax_t, *scale_ub) * (1/448), 1/(448*512)), result = e4m3(clamp(x * (1 / scale[t]))).
 * input bf16 (or fp16) [tokens, hidden] contiguous, hidden % 8 == 0, hidden <= 32768. */
int hb200_dynamic_per_token_scaled_fp8_quant(void* result, const void* input, void* scale, int64_t tokens,
                                             int64_t hidden, const float* scale_ub, int in_is_fp16, void* stream);

/* hb200_moe_build_schedule with every expert padded to a multiple of 256 rows (max_tiles, still in 128-row
 * units, must be even; ceil(pairs / 128) + 2 * experts always suffices), and hb200_nvfp4_grouped_matmul over
 * such a layout: 256 x 256 tiles on CTA pairs (cta_group::2), which halves the weight-tile traffic per CTA.
 * Falls back to the 128-row kernel where the pair kernel does not apply (N % 256 != 0, fp32 output). */
int hb200_moe_build_schedule_256(const int32_t* counts, int64_t experts, const int32_t* sorted_pairs, int64_t pairs,
                                 int32_t* padded_offsets, int32_t* tile_info, int64_t max_tiles,
                                 int32_t* row_of_sorted, int32_t* row_of_pair, void* stream);
int hb200_nvfp4_grouped_matmul_256(const void* a_packed, const void* b_packed, const void* scale_a,
                                   const void* scale_b, void* out, const int32_t* tile_info, int64_t max_m_tiles,
                                   int64_t n, int64_t k, int64_t groups, int64_t ldc, const float* row_scale,
                                   const float* group_alpha, float alpha, int out_dtype, void* stream);

/* Routing front-end of the MoE layer: softmax over the experts in fp32 (exp(x - max) / sum) followed by top-k,
 * one kernel (the reference's examples route with torch.softmax + torch.topk outside their kernels,
 * examples/moe_matmul_ogs.py:96-117 takes the result).  logits [tokens, experts] contiguous, logits_dtype
 * 0 bf16 / 1 fp16 / 2 fp32; weights [tokens, top_k] fp32 and chosen [tokens, top_k] int64 are written in
 * descending order of weight, equal weights by ascending expert index.  experts <= 1024, top_k <= experts. */
int hb200_moe_route_top_k(const void* logits, int logits_dtype, int64_t tokens, int64_t experts, int64_t top_k,
                          float* weights, int64_t* chosen, void* stream);

/* Stable sort of the (token, slot) pairs by expert plus the per-expert counts, on the device: what
 * moe_matmul_ogs_helion_kernel_args_gen computes with bincount + argsort and a host read
 * (examples/moe_matmul_ogs.py:96-117).  expert_of_pair: one entry per pair, int64 when idx_is_i64 != 0 (what
 * torch.topk returns), else int32; entries outside [0, experts) are dropped.  sorted_pairs [pairs] and
 * counts [experts] are written; scratch needs ceil(pairs / 1024) * experts int32.  experts <= 1024. */
int hb200_moe_sort_pairs(const void* expert_of_pair, int idx_is_i64, int64_t pairs, int64_t experts,
                         int32_t* sorted_pairs, int32_t* counts, int32_t* scratch, void* stream);

/* First expert GEMM of an NVFP4 MoE layer with the SiLU-mul in its epilogue (arguments as
 * hb200_nvfp4_grouped_matmul).  b_packed holds, per expert, n rows that interleave gate and up in blocks of
 * 128: rows [256 j, 256 j + 128) are gate outputs [128 j, 128 j + 128), rows [256 j + 128, 256 j + 256) the up
 * rows of the same outputs (n % 256 == 0).  Writes y = bf16(silu(gate) * up) to y_out [rows, n / 2] (leading
 * dimension ldy) and max |y[r, :]| to row_amax[r] (fp32 [max_m_tiles * 128], cleared by this call on the
 * stream).  Bit-identical to hb200_nvfp4_grouped_matmul + the silu_mul form of hb200_nvfp4_quantize_rows; it
 * saves writing and re-reading the [rows, n] intermediate.  The reference has no NVFP4 MoE
 * (examples/moe_matmul_ogs.py:31-85 is a bf16 top-1 GEMM); gate-first as in
 * pretuned_kernels/silu_and_mul_per_block_quant/silu_and_mul_per_block_quant.py:97-105. */
int hb200_nvfp4_grouped_matmul_silu(const void* a_packed, const void* b_packed, const void* scale_a,
                                    const void* scale_b, void* y_out, float* row_amax, const int32_t* tile_info,
                                    int64_t max_m_tiles, int64_t n, int64_t k, int64_t groups, int64_t ldy,
                                    const float* row_scale, const float* group_alpha, float alpha, void* stream);

/* The same call for a row layout whose groups are padded to multiples of 256 rows (hb200_moe_build_schedule_256;
 * max_m_tiles still counts 128-row tiles and is even): 256 x 256 tiles on CTA pairs, the same values bit for bit.
 * Shapes the pair kernel does not take run on the 128-row kernel.  No counterpart in the reference. */
int hb200_nvfp4_grouped_matmul_silu_256(const void* a_packed, const void* b_packed, const void* scale_a,
                                        const void* scale_b, void* y_out, float* row_amax, const int32_t* tile_info,
                                        int64_t max_m_tiles, int64_t n, int64_t k, int64_t groups, int64_t ldy,
                                        const float* row_scale, const float* group_alpha, float alpha, void* stream);

/* Per-token NVFP4 quantisation of rows whose maxima are already known (row_amax from the call above): row
 * r = row_idx[i] (i when null) of x [*, ldx] -> codes, swizzled scales, global_scale[r] = row_amax[r] / (6 * 448)
 * (times item_scale[i] in the stored copy).  Same codes and scales as hb200_nvfp4_quantize_rows. */
int hb200_nvfp4_quantize_rows_amax(const void* x_bf16, void* codes, void* scales_swizzled, float* global_scale,
                                   const float* row_amax, int64_t items, int64_t k, int64_t ldx,
                                   const int32_t* row_idx, const float* item_scale, void* stream);

/* ---- tensor-core GEMV / decode-batch skinny GEMM ----
 *
 * Same operators as hb200_nvfp4_gemv_bf16in / _fp4in (examples/nvfp4_gemv.py:432-525, batch rows 1..32 as in
 * the decode sweep), computed with tcgen05.mma on the packed weights so that no thread decodes a weight
 * byte.  bf16 activations are expanded into four NVFP4 residual terms first (error below 1e-3 of a
 * 16-element block's maximum, checked against the fp32 reference in the tests); NVFP4 activations are
 * used as they are.  Needs K % 32 == 0 (HB200_ERR_UNSUPPORTED otherwise: use the entry points above).
 *
 * `workspace` is caller-owned device memory of at least hb200_nvfp4_gemv_tc_workspace_bytes(...) bytes,
 * 256-byte aligned, zero-filled once before its first use (the kernels leave the part that must be zero
 * at zero again).  Calls that share a workspace must not overlap (same stream, or ordered by events);
 * HB200_ERR_WORKSPACE if it is too small.  out_ptrs / world / n_total / col0 as in the tensor-parallel
 * forms below; for a single GPU pass one pointer, world = 1, n_total = n, col0 = 0. */
int64_t hb200_nvfp4_gemv_tc_workspace_bytes(int64_t n, int64_t k, int64_t batch, int64_t terms);
int hb200_nvfp4_gemv_bf16in_tc(const void* weight_packed, const void* x_bf16, const void* weight_scale,
                               void* const* out_ptrs, int64_t world, int64_t n, int64_t k, int64_t batch,
                               int64_t n_total, int64_t col0, float alpha, void* workspace,
                               int64_t workspace_bytes, void* stream);
int hb200_nvfp4_gemv_fp4in_tc(const void* weight_packed, const void* x_packed, const void* weight_scale,
                              const void* x_scale, void* out_bf16, int64_t n, int64_t k, float alpha,
                              void* workspace, int64_t workspace_bytes, void* stream);

/* hb200_nvfp4_gemv_bf16in_tc for one GPU without a workspace argument, for callers that have no way to
 * obtain device memory at the point of the call.  The scratch is an 8 MiB array inside the library's device
 * image (one per device); this entry point and everything it calls allocate and free nothing, on the
 * device or through the caller's framework.  Limits: at most 8 activation rows and K <= 65536 always fit;
 * a shape whose workspace would exceed 8 MiB is refused with HB200_ERR_SCRATCH_LIMIT before anything runs.
 * The first call on a device (with that device current) looks the array up and clears its arrival counters
 * on `stream`: make that call during start-up, before any stream capture.  Calls on one device share the
 * array, so they must not overlap: issue them on one stream or order them with events, as two overlapping
 * calls would corrupt each other's partial sums.  Results are bit-identical to hb200_nvfp4_gemv_bf16in_tc.
 * No counterpart in the reference, whose kernels get their temporaries from torch's caching allocator. */
int hb200_nvfp4_gemv_bf16in_tc_builtin_scratch(const void* weight_packed, const void* x_bf16,
                                               const void* weight_scale, void* out_bf16, int64_t n, int64_t k,
                                               int64_t batch, float alpha, void* stream);

/* Re-zeroes, on `stream`, the tile arrival counters of the built-in scratch (the part that must be zero when a
 * call starts).  A call that ended with HB200_ERR_DEVICE_TIMEOUT, or two calls that overlapped on the device,
 * can leave counters non-zero, and every later call on that device would then leave output tiles unwritten
 * although hb200_device_status reads OK again: call this (or hb200_device_status(1), which does the same
 * synchronously when it clears a non-zero status) before going on.  Allocates nothing.  For a caller-owned
 * workspace the same holds: clear its first hb200_nvfp4_gemv_tc_counter_bytes() bytes. */
int hb200_nvfp4_gemv_tc_builtin_scratch_reset(void* stream);
int64_t hb200_nvfp4_gemv_tc_counter_bytes(void);

/* ---- tensor-parallel forms (one process per GPU, outputs in symmetric memory) ----
 *
 * The reference's distributed examples push results to peers from inside the kernel through symmetric
 * memory and signal pads (examples/distributed/all_gather_matmul.py:36-87,
 * helion/runtime/triton/dist_utils.py:291-406); these entry points are the same idea for the column-parallel
 * GEMV and GEMM: rank r owns weight rows [col0, col0 + n) of n_total, computes that slice of the output and
 * stores it into the [rows, n_total] buffer of every rank.  out_ptrs[i] is rank i's buffer as mapped into
 * this process (CUDA peer mapping of one symmetric allocation).  Peer memory is only ever stored to (plain
 * stores in the GEMV, bulk shared-to-global copies in the GEMM); no load and no multicast touches it. */
int hb200_nvfp4_gemv_bf16in_tp(const void* weight_packed, const void* x_bf16, const void* weight_scale,
                               void* const* out_ptrs, int64_t world, int64_t n, int64_t k, int64_t batch,
                               int64_t n_total, int64_t col0, float alpha, void* stream);

/* Row-parallel GEMV / skinny GEMM with a fused reduce-scatter (a K-sharded projection such as `down`): this rank
 * holds weight columns [N, K_local] and the matching activation columns, computes its fp32 partial of all N
 * outputs and stores the partial of output column c into the fp32 [world, batch, N / world] buffer of the rank
 * that owns c, at [this rank, row, c % (N / world)].  After hb200_peer_barrier, hb200_tp_reduce_partials adds the
 * partials of this rank's columns in rank order.  The pattern of examples/distributed/matmul_reduce_scatter.py:36-120,
 * with stores to the owners instead of loads from the peers.  N % world == 0. */
int hb200_nvfp4_gemv_bf16in_rs(const void* weight_packed, const void* x_bf16, const void* weight_scale,
                               void* const* partial_ptrs, int64_t world, int64_t rank, int64_t n, int64_t k_local,
                               int64_t batch, float alpha, void* stream);
int hb200_tp_reduce_partials(const void* partials_f32, void* out_bf16, int64_t world, int64_t batch, int64_t cols,
                             int64_t ld_out, void* stream);

/* ------------------------------------------------ dense bf16 / fp16 GEMM on CTA pairs and its fused collectives
 * c [M, N] = a [M, K] . b^T, b given K-major as [N, K]; pitches in elements; fp32 accumulate; 256 x 256 tiles on CTA
 * pairs with two accumulators in tensor memory.  M, N >= 256, 16-byte aligned a, b, c, lda % 8 == ldb % 8 ==
 * ldc % 8 == 0 (HB200_ERR_UNSUPPORTED otherwise).  The one-GPU form of the two calls below; stands where the
 * reference's distributed examples call a Helion matmul (examples/distributed/all_gather_matmul.py:95-141). */
int hb200_dense_matmul(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int64_t lda,
                       int64_t ldb, int64_t ldc, int is_bf16, void* stream);

/* All-gather + matmul (helion_all_gather_matmul, examples/distributed/all_gather_matmul.py:145-196):
 * c [world * rows_local, N] = gathered a . b^T.  a_shard: this rank's rows [rows_local, K], contiguous.
 * gather_ptrs[i] / progress_ptrs[i]: rank i's gather buffer [world * rows_local, K] (contiguous) and its progress
 * counters (uint32 [world * splits], zero before the first call, never reset), as mapped into this process
 * (symmetric memory); entry `rank` is this rank's own.  The GEMM takes the row tiles in arrival order (own rows
 * first, read from a_shard itself) and waits (bounded, system-scope acquire) for a chunk's counter before the first
 * load of its rows.  call_number counts the calls on this buffer set from 1.  Two ways to fill the buffers:
 *  - push != 0, one kernel does everything: the two warps of every CTA that have no role in the GEMM copy this
 *    rank's shard, in `splits` chunks, into every peer's buffer (stores to peer memory only) and add one arrival per
 *    warp to the chunk's counter there; a chunk has landed when its counter reads (pushing warps) * call_number.
 *    All ranks call with the same shapes and call_number.
 *  - push == 0, the reference's structure: somebody else (copy engines on another stream) fills this rank's buffer
 *    chunk by chunk and, after a chunk, writes call_number into its counter (e.g. a stream memory write); only
 *    entry `rank` of the two pointer arrays is read.
 * Either way the caller puts a barrier between calls (a rank must not overwrite a buffer that is still being
 * read).  (rows_local / splits) % 256 == 0, K % 8 == 0, N >= 256, ldc % 8 == 0. */
int hb200_ag_matmul(const void* a_shard, void* const* gather_ptrs, void* const* progress_ptrs, const void* b, void* c,
                    int64_t rows_local, int64_t n, int64_t k, int64_t ldb, int64_t ldc, int64_t world, int64_t rank,
                    int64_t splits, uint32_t call_number, int push, int is_bf16, void* stream);

/* Matmul + reduce-scatter, first half (matmul_reduce_scatter_kernel, examples/distributed/matmul_reduce_scatter.py:
 * 37-115): a [M, K_local] . b^T (b K-major [N, K_local]) is this rank's partial product; the epilogue rounds it to the
 * operand type and stores rows [d R, d R + R), R = M / world, into slot `rank` of recv_ptrs[d], rank d's receive
 * buffer [world, R, N] (contiguous, symmetric memory), with TMA stores; nothing is loaded from peer memory.
 * M % (256 * world) == 0, N % 8 == 0, N >= 256.  Follow with hb200_peer_barrier and hb200_reduce_slots. */
int hb200_matmul_rs(const void* a, const void* b, void* const* recv_ptrs, int64_t m, int64_t n, int64_t k, int64_t lda,
                    int64_t ldb, int64_t world, int64_t rank, int is_bf16, void* stream);

/* Second half: out [rows, cols] (row pitch ld_out) = cast(sum over s, ascending, of fp32(slots[s, rows, cols])).
 * The order is fixed, so results do not depend on timing.  cols % 8 == 0, ld_out % 8 == 0, 16-byte aligned. */
int hb200_reduce_slots(const void* slots, void* out, int64_t world, int64_t rows, int64_t cols, int64_t ld_out,
                       int is_bf16, void* stream);

/* out_dtype 0 = bf16, 1 = fp16.  Needs m >= 256, n >= 256, K % 32 == 0, n_total % 8 == 0, col0 % 8 == 0
 * (HB200_ERR_UNSUPPORTED otherwise: compute locally and gather with a collective). */
int hb200_nvfp4_scaled_matmul_tp(const void* a_packed, const void* b_packed, const void* scale_a,
                                 const void* scale_b, void* const* out_ptrs, int64_t world, int64_t rank,
                                 int64_t m, int64_t n, int64_t k, int64_t n_total, int64_t col0, float alpha,
                                 int out_dtype, void* stream);

/* ---- expert-parallel exchange of the NVFP4 MoE layer (one process per GPU) ----
 *
 * Rank r owns experts [r E/W, (r+1) E/W) and `tokens` tokens of its own.  Every rank allocates one symmetric,
 * zero-filled buffer of hb200_ep_buffer_bytes(...) bytes; bases[i] is rank i's buffer as mapped into this process.
 * A step: hb200_ep_dispatch, hb200_peer_barrier, [hb200_ep_collect, sort + schedule, hb200_ep_gather, the two grouped
 * GEMMs], hb200_ep_return, hb200_peer_barrier, hb200_ep_combine.  Rows travel as NVFP4 (codes + block scales + one
 * global scale per token), results as ONE routing-weighted row per (token, expert rank), fp16 values with a power-of-two row factor.  The receive areas
 * have a capacity that follows from the shapes (tokens * min(top_k, E/W) pairs per source), so no count is ever
 * read on the host.  Peer memory is only stored to; nothing is multicast.  hidden % 64 == 0, hidden <= 8192, experts % world == 0.
 * No counterpart in the reference (its distributed examples push to peers and signal the same way:
 * examples/distributed/all_gather_matmul.py:36-87). */
int64_t hb200_ep_buffer_bytes(int64_t world, int64_t tokens, int64_t hidden, int64_t top_k, int64_t experts);
int64_t hb200_ep_slots(int64_t world, int64_t tokens, int64_t hidden, int64_t top_k, int64_t experts);
/* codes_t [T, H/2], scales_t swizzled [T, H/16], g_t [T]: per-token NVFP4 rows (hb200_nvfp4_quantize); weights fp32
 * and experts_of_pair int64 [T * top_k] (hb200_moe_route_top_k); sorted_pairs / counts from hb200_moe_sort_pairs over
 * the global expert ids; route_local int32 [T * top_k] (this rank's memory) receives where every pair went. */
int hb200_ep_dispatch(const void* codes_t, const void* scales_t, const float* g_t, const float* weights,
                      const int64_t* experts_of_pair, const int32_t* sorted_pairs, const int32_t* counts,
                      int32_t* route_local, void* const* bases, int64_t world, int64_t rank, int64_t tokens,
                      int64_t hidden, int64_t top_k, int64_t experts, void* stream);
/* expert_of_slot int32 [hb200_ep_slots]: local expert of every receive slot, -1 where nothing arrived. */
int hb200_ep_collect(const void* base, int32_t* expert_of_slot, int64_t world, int64_t rank, int64_t tokens,
                     int64_t hidden, int64_t top_k, int64_t experts, void* stream);
/* Received rows -> padded expert-sorted operand of the first grouped GEMM; w_row = routing weight per padded row.
 * sorted_slots / row_of_sorted from hb200_moe_sort_pairs / hb200_moe_build_schedule over expert_of_slot. */
int hb200_ep_gather(const void* base, const int32_t* sorted_slots, const int32_t* row_of_sorted, void* codes_out,
                    void* scales_out, float* g_out, float* w_row, int64_t world, int64_t rank, int64_t tokens,
                    int64_t hidden, int64_t top_k, int64_t experts, void* stream);
/* o [padded rows, H] bf16: the second grouped GEMM's rows; row_of_slot: padded row of every receive slot. */
int hb200_ep_return(const void* o_bf16, int64_t ldo, const int32_t* row_of_slot, const float* w_row,
                    void* const* bases, int64_t world, int64_t rank, int64_t tokens, int64_t hidden, int64_t top_k,
                    int64_t experts, void* stream);
int hb200_ep_combine(const void* base, const int32_t* route_local, void* out_bf16, int64_t world, int64_t rank,
                     int64_t tokens, int64_t hidden, int64_t top_k, int64_t experts, void* stream);

/* Barrier between the ranks as a kernel on `stream`: flag_ptrs[i] is rank i's array of >= world uint32
 * (zero-initialised symmetric memory), epoch_counter one uint32 in this rank's own memory (zero-initialised,
 * owned by the barrier).  Orders every earlier peer store on the stream before the other ranks' later reads.
 * The wait is bounded; on expiry hb200_device_status reports HB200_ERR_DEVICE_TIMEOUT.  Replaces the
 * signal-pad barrier of helion/runtime/triton/dist_utils.py:291-406. */
int hb200_peer_barrier(void* const* flag_ptrs, int64_t world, int64_t rank, void* epoch_counter, void* stream);

/* Sticky device-side status: HB200_OK, or HB200_ERR_DEVICE_TIMEOUT once a
 * kernel gave up a bounded wait (its outputs are then undefined).  reset != 0
 * clears it.  Synchronises the device; not for use on the hot path.  (No
 * counterpart in the reference, whose device waits are unbounded.) */
int hb200_device_status(int reset);

/* Budget, in SM clock cycles, of every bounded device-side wait of the library on the current device (the
 * mbarrier waits of the tcgen05 pipelines and the flag wait of hb200_peer_barrier); default 4e9, about two
 * seconds.  Synchronous; do not call while kernels of the library are in flight.  (The reference's waits are
 * unbounded: helion/runtime/triton/dist_utils.py:175-193.) */
int hb200_set_wait_budget_cycles(int64_t cycles);

/* Launches one CTA that waits, with the bounded wait every pipeline uses, on an mbarrier nothing arrives on:
 * the wait runs out after one budget, the kernel returns and hb200_device_status reads
 * HB200_ERR_DEVICE_TIMEOUT until reset.  Exercises the expiry path without a fault; shorten the budget first. */
int hb200_selftest_bounded_wait(void* stream);

/* Self-test of the short exact reciprocal and division the quant producers use where the divisor's range is
 * known (no reference counterpart).  `mismatches` points at three 64-bit device counters: [0] counts the fp32
 * divisors in [2^-100, 2^125], all of which are tried, whose short reciprocal differs from the IEEE one; [1] the
 * quotients of the one-correction-step division that differ from the IEEE quotient among four numerators per
 * divisor (|x| >= 2^-100); [2] the same for two correction steps.  All read 0 when the short forms are exact. */
int hb200_selftest_exact_reciprocal(unsigned long long* mismatches, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HELION_B200_H_ */
