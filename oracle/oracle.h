/*
 * TEST INFRASTRUCTURE ONLY.  Scalar host restatement of the W8A8 (i8i8) linear
 * path of OpenPPL/ppl.llm.kernel.cuda.  It is the checker for the CUDA kernels
 * and the timed CPU baseline; nothing in the product library links or calls it.
 *
 * Parity status: the reference ships no golden vectors or result-checking tests
 * for this path (its test/ directory only times GEMMs).  The restatement is
 * therefore pinned against outputs of the reference's own kernels, compiled
 * unmodified into oracle/_ref and run on the GPU (tests/test_reference_parity.py
 * and the fixtures under tests/golden/ that were produced by such a run).
 *
 * Every function cites the reference file:line it follows (paths relative to
 * the reference project root).
 */
#ifndef PPLB200_ORACLE_H
#define PPLB200_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* matrix_layout_t values: include/ppl/kernel/llm/cuda/common/matrix_layout.h:25-31 */
enum {
    ORC_LAYOUT_ROW_MAJOR    = 0,
    ORC_LAYOUT_COL_MAJOR    = 1,
    ORC_LAYOUT_COL32        = 2,
    ORC_LAYOUT_COL32_2R_4R4 = 3,
    ORC_LAYOUT_COL4_4R2_8C  = 4
};

/* IEEE binary16 <-> binary32/64 conversions, round-to-nearest-even, bit level. */
uint16_t orc_f32_to_f16(float f);
uint16_t orc_f64_to_f16(double d);
float    orc_f16_to_f32(uint16_t h);
/* fp16 + fp16 with one rounding (the device's native half add). */
uint16_t orc_f16_add(uint16_t a, uint16_t b);

/* (row, col) -> element offset for each layout; matrix_layout.h:34-142 */
int64_t orc_layout_offset(int32_t layout, int64_t rows, int64_t cols, int64_t row, int64_t col);

/* Number of worker threads used by the bulk functions below (default 1). */
void    orc_set_threads(int32_t n);
int32_t orc_get_threads(void);

/* pmx/i8i8/quantize.cu:27-80 (kernel), :82-124 (launcher). Returns 0, or 2 (unsupported layout). */
int32_t orc_minmax_quantize_fp16(const uint16_t* x, int64_t batch, int64_t quant_dim, float up_scale,
                                 int32_t to_layout, int8_t* q, uint16_t* scale);

/* cublas/gemm.cu:171-194 as called from pmx/i8i8/column_parallel_linear.cu:96-119:
 * C[M,N] (i32, ldc) = A[M,K] (i8, lda) * B[N,K]^T (i8, ldb). */
void orc_gemm_i8i8i32(const int8_t* A, int64_t lda, const int8_t* B, int64_t ldb,
                      int64_t M, int64_t N, int64_t K, int32_t* C, int64_t ldc);
/* Same product restricted to rows [m0, m1) of A/C (used for sampled checks of big shapes). */
void orc_gemm_i8i8i32_rows(const int8_t* A, int64_t lda, const int8_t* B, int64_t ldb,
                           int64_t m0, int64_t m1, int64_t N, int64_t K, int32_t* C, int64_t ldc);

/* pmx/i8i8/quantize.cu:126-169 (kernel), :171-234 (launcher). Returns 0, 4 (N % 4) or 2 (layout). */
int32_t orc_minmax_dequantize_fp16(const int32_t* acc, const uint16_t* bias, const uint16_t* scale_m,
                                   const uint16_t* scale_n, int64_t batch, int64_t quant_dim,
                                   float down_m, float down_n, int32_t from_layout, uint16_t* out);

/* Whole path on one device: quantize -> GEMM -> dequant(+bias) [-> re-quantize].
 * Any of xq, sm, acc, yq, yq_scale may be NULL (then not returned / not computed).
 * Re-quantize = orc_minmax_quantize_fp16 applied to the fp16 output. */
int32_t orc_w8a8_linear(const uint16_t* x, const int8_t* w, const uint16_t* scale_n, const uint16_t* bias,
                        int64_t M, int64_t N, int64_t K, float up_scale, float down_m, float down_n,
                        float requant_up_scale,
                        int8_t* xq, uint16_t* sm, int32_t* acc, uint16_t* y, int8_t* yq, uint16_t* yq_scale);

/* pmx/i8i8/rms_norm.cu:40-182 (kernels), :186-302 (launcher); pmx/quant_utils.h:75-92 (quant_scalar).
 * z = input + skip (fp16 add) -> skip_out; r = 1/sqrt(mean(z^2) + eps); amax = max(eps, max|z*w|);
 * scale = max(amax * r / 127, 1e-7); q = clamp(round_half_away((z*w*r) * (1/scale)), -127, 127).
 * The sum of squares is taken in double and the reciprocal square root exactly, whereas the device
 * kernels sum in fp32 (order unspecified) and use the approximate rsqrtf: compare with tolerance
 * (scale within 1 fp16 ulp, int8 within 1).  Returns 0, or 2 (unsupported layout). */
int32_t orc_skip_rmsnorm_minmax_quantize_fp16(const uint16_t* input, const uint16_t* weight, const uint16_t* skip,
                                              float eps, int64_t batch, int64_t dim, float up_scale, int32_t to_layout,
                                              uint16_t* skip_out, uint16_t* out_scale, int8_t* q);

/* pmx/i8i8/silu.cu:44-133 / swiglu.cu:42-128: dequantize -> SiLU [x gate] or SwiGLU -> fp16 workspace;
 * row max of the fp32 value before rounding; q = rn(float(fp16) / scale).  kind 0 SiLU, 1 gated SiLU
 * (gate int32 [batch, dim] with its own scales), 2 SwiGLU (input [batch, 2 dim] = [x | gate], channel
 * scales [2 dim]).  expf is exact here, the device uses __expf: compare with tolerance.  out_q / out_scale
 * may be NULL (dequantize + activation only).  Row-major only. */
int32_t orc_activation_requantize(int32_t kind, const int32_t* input, const uint16_t* scale_b, const uint16_t* scale_c,
                                  const int32_t* gate, const uint16_t* gate_scale_b, const uint16_t* gate_scale_c,
                                  int64_t batch, int64_t dim, float beta, float up_scale, float down_b, float down_c,
                                  uint16_t* workspace, int8_t* out_q, uint16_t* out_scale);

/* pmx/i8i8/split.cu:44-84: dequantize (+bias) and route 4-column groups to three row-major outputs. */
int32_t orc_dequantize_split3(const int32_t* acc, const uint16_t* bias, const uint16_t* scale_m, const uint16_t* scale_n,
                              int64_t batch, int64_t dim, int64_t d0, int64_t d1, int64_t d2, float down_m, float down_n,
                              uint16_t* o0, uint16_t* o1, uint16_t* o2);

/* Elementwise sum of `parts` int32 partial accumulators (row-parallel reduction, exact). */
void orc_sum_partials_i32(const int32_t* const* parts, int32_t nparts, int64_t count, int32_t* out);

#ifdef __cplusplus
}
#endif
#endif
