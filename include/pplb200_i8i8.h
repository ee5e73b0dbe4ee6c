/*
 * C ABI of the B200 (sm_100a) W8A8 "i8i8" linear path.
 *
 * Every entry point is stream-ordered and asynchronous, allocates nothing, and
 * returns a ppl.common RetCode value (0 success, 2 unsupported, 4 invalid value,
 * 10 device runtime error).  All pointers are device pointers unless a comment
 * says otherwise; the caller owns every buffer, stream and communicator.
 * Matrix layouts use the reference's matrix_layout_t numbering
 * (include/ppl/kernel/llm/cuda/common/matrix_layout.h:25-31).
 *
 * The C++ operator API of the reference (namespace ppl::kernel::llm::cuda) is
 * provided on top of this ABI as header-inline forwards under
 * include/ppl/kernel/llm/cuda/, so no C++ ABI crosses the shared library.
 */
#ifndef PPLB200_I8I8_H
#define PPLB200_I8I8_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

typedef struct CUstream_st* pplb200_stream_t; /* == cudaStream_t */

/* epilogue modes of pplb200_i8i8_gemm */
enum {
    PPLB200_EPI_RAW_I32 = 0,          /* out = int32 accumulators [M, N]                                  */
    PPLB200_EPI_DEQUANT_F16 = 1,      /* out = fp16 (acc * scale_N * down_N * scale_M * down_M) + bias   */
    PPLB200_EPI_DEQUANT_F16_REQUANT_I8 = 2 /* as 1, plus out_q/out_q_scale = per-token quantize(out)    */
};

/* Library / build identification: "pplb200 i8i8 <version> sm_100a". */
const char* pplb200_version(void);

/* Last error text recorded by a failing call on the calling thread ("" if none). */
const char* pplb200_last_error(void);

/*
 * Per-token dynamic symmetric quantizer, fp16 -> int8.
 * Replaces ppl::kernel::llm::cuda::pmx::i8i8::minmax_quantize_fp16
 *   (include/ppl/kernel/llm/cuda/pmx/i8i8/quantize.h:32-41; src/.../pmx/i8i8/quantize.cu:27-124).
 * in fp16 [batch, quant_dim] row-major; q int8 [batch, quant_dim] in `to_layout`
 * (ROW_MAJOR, COL32 or COL32_2R_4R4); scale fp16 [batch] = scale * up_scale.
 * Requires quant_dim % 16 == 0 and 16-byte aligned in/q.
 */
int32_t pplb200_i8i8_minmax_quantize_fp16(pplb200_stream_t stream, const void* in, int64_t batch, int64_t quant_dim,
                                          float up_scale, int32_t to_layout, void* q, void* scale);

/*
 * int32 -> fp16 dequantize with row scale x column scale and optional fp16 bias.
 * Replaces ppl::kernel::llm::cuda::pmx::i8i8::minmax_dequantize_fp16
 *   (include/.../pmx/i8i8/quantize.h:43-55; src/.../pmx/i8i8/quantize.cu:126-234).
 * acc int32 [batch, quant_dim] in `from_layout` (any of the five layouts); out fp16 row-major.
 * Requires quant_dim % 4 == 0 (RC_INVALID_VALUE otherwise, as the reference).
 */
int32_t pplb200_i8i8_minmax_dequantize_fp16(pplb200_stream_t stream, const void* acc, const void* optional_bias,
                                            const void* scale_per_batch, const void* scale_per_channel,
                                            int64_t batch, int64_t quant_dim, float down_scale_batch,
                                            float down_scale_channel, int32_t from_layout, void* out);

/*
 * Fused skip-add + RMSNorm + per-token quantize: the producer that feeds the linear in a block.
 * Replaces ppl::kernel::llm::cuda::pmx::i8i8::skip_rmsnorm_minmax_quantize_fp16
 *   (include/.../pmx/i8i8/quantize.h:128-141; src/.../pmx/i8i8/rms_norm.cu:40-302).
 * input, optional_skip fp16 [batch, normalize_shape]; weight fp16 [normalize_shape];
 * skip_out fp16 [batch, normalize_shape] = input + skip; output int8 in `to_layout` (ROW_MAJOR, COL32,
 * COL32_2R_4R4); output_scale fp16 [batch] = scale * up_scale.  normalize_shape % 16 == 0, <= 32768.
 * Rounding: half away from zero with a clamp to +-127, as the reference's quant_scalar.
 */
int32_t pplb200_i8i8_skip_rmsnorm_minmax_quantize_fp16(pplb200_stream_t stream, const void* input, const void* weight,
                                                       const void* optional_skip, float eps, int64_t batch,
                                                       int64_t normalize_shape, float up_scale, int32_t to_layout,
                                                       void* skip_out, void* output_scale, void* output);

/*
 * Consumers of the raw int32 accumulators (column_parallel_linear with gather_output == 0).
 * Replace, with the same argument meaning,
 *   minmax_dequantize_split3_fp16   (include/.../pmx/i8i8/quantize.h:57-74;  src/.../pmx/i8i8/split.cu:44-169)
 *   minmax_dequantize_silu_fp16     (quantize.h:76-90; declared by the reference, defined nowhere in it)
 *   minmax_requantize_silu_fp16     (quantize.h:92-109; src/.../pmx/i8i8/silu.cu:44-199)
 *   minmax_requantize_swiglu_fp16   (quantize.h:111-126; src/.../pmx/i8i8/swiglu.cu:42-185)
 * input int32 [batch, quant_dim] (SwiGLU: [batch, 2 * quant_dim] = [x | gate], channel scales [2 * quant_dim]).
 * Activations: layouts ROW_MAJOR, COL32, COL32_2R_4R4; quant_dim % 16 == 0 and <= 32768; `workspace`
 * receives the fp16 activated values (may be NULL), `output` int8 and `scale` fp16 [batch] = scale * up_scale.
 * split3: any of the five layouts, quant_dim and the three split sizes multiples of 4.
 */
int32_t pplb200_i8i8_minmax_dequantize_split3_fp16(pplb200_stream_t stream, const void* input, const void* optional_bias,
                                                   const void* scale_per_batch, const void* scale_per_channel,
                                                   int64_t batch, int64_t quant_dim, int64_t split_dim_0,
                                                   int64_t split_dim_1, int64_t split_dim_2, float down_scale_batch,
                                                   float down_scale_channel, int32_t from_layout, void* output_0,
                                                   void* output_1, void* output_2);
int32_t pplb200_i8i8_minmax_dequantize_silu_fp16(pplb200_stream_t stream, const void* input, const void* input_scale_per_batch,
                                                 const void* input_scale_per_channel, const void* optional_gate,
                                                 const void* gate_scale_per_batch, const void* gate_scale_per_channel,
                                                 int64_t batch, int64_t quant_dim, int32_t from_layout,
                                                 float down_scale_batch, float down_scale_channel, void* output);
int32_t pplb200_i8i8_minmax_requantize_silu_fp16(pplb200_stream_t stream, const void* input, const void* input_scale_per_batch,
                                                 const void* input_scale_per_channel, const void* optional_gate,
                                                 const void* gate_scale_per_batch, const void* gate_scale_per_channel,
                                                 int64_t batch, int64_t quant_dim, int32_t layout, float up_scale,
                                                 float down_scale_batch, float down_scale_channel, void* workspace,
                                                 void* output, void* scale);
int32_t pplb200_i8i8_minmax_requantize_swiglu_fp16(pplb200_stream_t stream, const void* input, const void* input_scale_per_batch,
                                                   const void* input_scale_per_channel, int64_t batch, int64_t quant_dim,
                                                   float beta, int32_t layout, float up_scale, float down_scale_batch,
                                                   float down_scale_channel, void* workspace, void* output, void* scale);

/*
 * Fused gate+up projection: GEMM + dequantize + SwiGLU + per-token re-quantize in one pass over the
 * accumulators (they never leave tensor memory as int32).  Same result, bit for bit, as
 * column_parallel_linear(gather_output = false) followed by minmax_requantize_swiglu_fp16
 *   (src/.../pmx/i8i8/column_parallel_linear.cu:81-85,136; src/.../pmx/i8i8/swiglu.cu:42-185),
 * which is how the reference runs this layer (two kernels and a 4 * M * 2 * act_dim byte round trip).
 * input int8 [M, K] (row stride lda); weight int8 [2 * act_dim, K] = [x rows | gate rows];
 * scale_N fp16 [2 * act_dim]; activated fp16 [M, act_dim] (the reference's `workspace`);
 * out_q int8 [M, act_dim]; out_q_scale fp16 [M].  ws: pplb200_i8i8_gate_up_swiglu_workspace_bytes().
 * Shapes that cannot use the fused kernel (M <= 128, act_dim % 128 != 0, too few tiles) run the two
 * steps separately inside this call (the workspace size accounts for the int32 buffer).
 */
int64_t pplb200_i8i8_gate_up_swiglu_workspace_bytes(int64_t M, int64_t act_dim, int64_t K);
int32_t pplb200_i8i8_gate_up_swiglu_requant(pplb200_stream_t stream, const void* input, int64_t lda, const void* weight,
                                            int64_t M, int64_t act_dim, int64_t K, const void* scale_M,
                                            const void* scale_N, float beta, float up_scale, float down_scale_M,
                                            float down_scale_N, void* ws, int64_t ws_bytes, void* activated,
                                            void* out_q, void* out_q_scale);

/*
 * Scratch bytes pplb200_i8i8_gemm asks for (M, N, K, mode): the row maxima of mode 2 (required: M * 4 rounded up to
 * 256) and, for M > 128, about 10.5 MB through which the CTA pairs of the large-batch kernel exchange K slices of
 * the few tiles left over when the tile count is not a multiple of the pair count (optional: a NULL or smaller
 * workspace only switches that off; results are the same, the GEMM is up to one wave of tiles slower).  256-byte
 * aligned, contents need not be initialised, not shared by calls that may run at the same time.  0 means `ws` may be
 * NULL.
 */
int64_t pplb200_i8i8_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t epilogue_mode);

/*
 * C[M,N] = A[M,K] (int8, row-major, lda) x B[N,K]^T (int8, row-major, ldb) on tcgen05 tensor
 * cores with int32 TMEM accumulators, plus the fused epilogue selected by `epilogue_mode`.
 * Replaces ppl::kernel::llm::cuda::cublas::gemm_i8i8i32
 *   (include/.../cublas/gemm.h:56-79; src/.../cublas/gemm.cu:171-363) and, for modes 1/2, the
 *   minmax_dequantize_fp16 launch that follows it in the linear ops
 *   (src/.../pmx/i8i8/column_parallel_linear.cu:136-157).
 * Requires K % 16 == 0, lda % 16 == 0, ldb % 16 == 0, N % 8 == 0, 16-byte aligned A, B, out.
 * out: int32 [M, ldc] (mode 0) or fp16 [M, ldc] (modes 1, 2).
 * Mode 2 also writes out_q int8 [M, N] and out_q_scale fp16 [M] = scale * requant_up_scale, where
 * (out_q, scale) = per-token quantize of the fp16 `out` rows; it needs `ws` of
 * pplb200_i8i8_gemm_workspace_bytes() bytes (contents need not be initialised).
 */
int32_t pplb200_i8i8_gemm(pplb200_stream_t stream, const void* A, int64_t lda, const void* B, int64_t ldb,
                          int64_t M, int64_t N, int64_t K, int32_t epilogue_mode,
                          const void* scale_M, const void* scale_N, const void* optional_bias,
                          float down_scale_M, float down_scale_N, float requant_up_scale,
                          void* ws, int64_t ws_bytes, void* out, int64_t ldc, void* out_q, void* out_q_scale);

/*
 * C[M,N] (int32, ldc) = alpha * (A[M,K] x B[N,K]^T) + beta * C + optional_bias_i32[n], in wrapping int32
 * arithmetic: the full contract of ppl::kernel::llm::cuda::cublas::gemm_i8i8i32 (int32 alpha / beta and the
 * int32 bias epilogue; include/ppl/kernel/llm/cuda/cublas/gemm.h:56-79, src/.../cublas/gemm.cu:187-188,239-243,329-345).
 * With alpha = 1, beta = 0 and no bias it is pplb200_i8i8_gemm in RAW_I32 mode.  beta != 0 reads C before it
 * is overwritten.  Same shape and alignment rules as pplb200_i8i8_gemm; the bias pointer 16-byte aligned.
 */
int32_t pplb200_i8i8_gemm_i32(pplb200_stream_t stream, const void* A, int64_t lda, const void* B, int64_t ldb,
                              int64_t M, int64_t N, int64_t K, int32_t alpha, int32_t beta, const void* optional_bias_i32,
                              void* C, int64_t ldc);

/*
 * Same result as pplb200_i8i8_gemm with PPLB200_EPI_DEQUANT_F16_REQUANT_I8 (out fp16 [M,N] with
 * ldc == N, out_q int8 [M,N], out_q_scale fp16 [M]) but WITHOUT a workspace argument and without
 * allocating anything: the per-row scratch lives in a fixed array inside the library.
 * This entry point has no counterpart in the reference (whose linears take caller-provided buffers
 * for everything); it exists for callers that cannot obtain device memory when they need the op --
 * runtimes that gave all of HBM to their own pool and forbid cudaMalloc afterwards, or code running
 * where the CUDA allocation calls are not allowed.
 * Limits and rules: M <= PPLB200_STATIC_SCRATCH_MAX_ROWS (larger M returns RC_INVALID_VALUE); the
 * array (64 KiB) stays resident on every GPU that loads the library; all calls on a device share
 * it, so calls whose GPU work overlaps race -- issue them on one stream or order them; the first
 * call on a device resolves the array's address, so make it before any stream capture starts.
 */
#define PPLB200_STATIC_SCRATCH_MAX_ROWS 16384
int32_t pplb200_i8i8_gemm_requant_static_scratch(pplb200_stream_t stream, const void* A, int64_t lda, const void* B,
                                                 int64_t ldb, int64_t M, int64_t N, int64_t K,
                                                 const void* scale_M, const void* scale_N, const void* optional_bias,
                                                 float down_scale_M, float down_scale_N, float requant_up_scale,
                                                 void* out, void* out_q, void* out_q_scale);

/*
 * Scratch bytes pplb200_i8i8_linear_fp16 needs (quantized activations, row scales, GEMM scratch).
 */
int64_t pplb200_i8i8_linear_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t epilogue_mode);

/*
 * Whole single-device path: y = dequant( quantize(x) x W^T ) (+ bias) [-> re-quantize].
 * x fp16 [M,K]; W int8 [N,K] row-major; scale_N fp16 [N] (up-scaled by 1/down_scale_N); bias fp16 [N] or NULL.
 * Equivalent to minmax_quantize_fp16 followed by column_parallel_linear(gather_output = true, size 1)
 *   (src/.../pmx/i8i8/quantize.cu:82; src/.../pmx/i8i8/column_parallel_linear.cu:29-182).
 * epilogue_mode is PPLB200_EPI_DEQUANT_F16 or PPLB200_EPI_DEQUANT_F16_REQUANT_I8.
 */
int32_t pplb200_i8i8_linear_fp16(pplb200_stream_t stream, const void* x, const void* W, const void* scale_N,
                                 const void* optional_bias, int64_t M, int64_t N, int64_t K,
                                 float up_scale, float down_scale_M, float down_scale_N,
                                 int32_t epilogue_mode, float requant_up_scale,
                                 void* ws, int64_t ws_bytes, void* y, void* y_q, void* y_q_scale);

/*
 * The same fused linear for callers whose activations and results live in HOST memory (pinned for the copies to be
 * asynchronous): x_host fp16 [M, K] in, y_host fp16 [M, N] out (and y_q_host int8 [M, N], y_q_scale_host fp16 [M]
 * with the re-quantize epilogue).  The batch is cut into chunks of `chunk_rows` tokens (0: 1024) and the three steps
 * of consecutive chunks -- host -> device copy, quantize + GEMM + epilogue on `stream`, device -> host copy -- run on
 * three streams at once (the two copy streams and their events are created per device at the first call, which
 * therefore should come before any stream capture), so a large batch costs little more than its slower copy
 * direction; with chunks of 1024 tokens or more the first chunk goes in as chunk_rows / 8, / 8, / 4 and / 2 tokens, so
 * that the copy out, usually the longest of the three, starts early.  Chunking is exact: the per-token quantizer and
 * the epilogue work row by row.  `ws` is DEVICE memory of
 * pplb200_i8i8_linear_host_workspace_bytes (two sets of staging buffers); weights, scales and bias are device
 * pointers as in pplb200_i8i8_linear_fp16.  Work enqueued on `stream` after the call runs after the last copy out.
 * No counterpart in the reference, whose operators take device pointers only.
 */
int64_t pplb200_i8i8_linear_host_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t epilogue_mode, int64_t chunk_rows);
int32_t pplb200_i8i8_linear_fp16_host(pplb200_stream_t stream, const void* x_host, const void* W, const void* scale_N,
                                      const void* optional_bias, int64_t M, int64_t N, int64_t K, float up_scale,
                                      float down_scale_M, float down_scale_N, int32_t epilogue_mode, float requant_up_scale,
                                      int64_t chunk_rows, void* ws, int64_t ws_bytes, void* y_host, void* y_q_host,
                                      void* y_q_scale_host);

/*
 * Tensor-parallel linears.  `nccl_comm` is an ncclComm_t (may be NULL when size == 1).
 *
 * Column parallel: replaces ppl::kernel::llm::cuda::pmx::i8i8::column_parallel_linear
 *   (include/.../pmx/i8i8/column_parallel_linear.h:33-58; src/.../pmx/i8i8/column_parallel_linear.cu:29-182).
 * input int8 [M,K]; weight int8 [N/size, K]; scale_N / bias are the rank's slices.
 * gather_output == 0: `output` receives RAW int32 [M, N/size] (no dequant), as the reference.
 * gather_output != 0: fp16; size == 1 -> output [M,N]; size > 1 -> all-gather into gather_buffer
 *   [size, M, N/size] then transpose to output [M, N].  quant_buffer is unused (the int32
 *   accumulators never leave the chip) but accepted.
 * weight_layout ROW_MAJOR: operands as above.  COL32_2R_4R4 / COL4_4R2_8C (the Turing / Ampere tensor-core orders
 *   the reference hands to gemm_i8i8i32_col32, src/.../pmx/i8i8/column_parallel_linear.cu:66-75,120-131): `input`
 *   is then COL32 [M, K], the weight is in that order, and with gather_output == 0 the raw int32 output is COL32
 *   [M, N/size], exactly as the reference leaves them.  sm_100a's tensor cores read none of these orders, so both
 *   operands are first re-laid out into `ws`, which must then hold
 *   roundup(M*K, 256) + roundup(N/size*K, 256) (+ roundup(M*N/size*4, 256) when gather_output == 0) bytes, 256-byte
 *   aligned (RC_UNSUPPORTED with the needed size in pplb200_last_error otherwise); K % 32 == 0, (N/size) % 32 == 0.
 *   Converting the weights once at load time with pplb200_i8i8_relayout and passing ROW_MAJOR avoids that pass.
 */
int32_t pplb200_i8i8_column_parallel_linear(pplb200_stream_t stream, const void* input, int64_t M,
                                            const void* weight, const void* optional_bias,
                                            const void* scale_M, const void* scale_N,
                                            float down_scale_M, float down_scale_N,
                                            int64_t in_features, int64_t out_features, int32_t weight_layout,
                                            int32_t rank, int32_t size, void* nccl_comm,
                                            int32_t gather_output, void* gather_buffer, void* quant_buffer,
                                            void* ws, int64_t ws_bytes, void* output);

/*
 * Row parallel: replaces ppl::kernel::llm::cuda::pmx::i8i8::row_parallel_linear
 *   (include/.../pmx/i8i8/row_parallel_linear.h:33-58; src/.../pmx/i8i8/row_parallel_linear.cu:28-162).
 * input int8 [M, K/size] with `input_ld` bytes between rows (K/size when the shard is contiguous, as in
 *   the reference; K when it is a column slice of the full quantized activation [M, K]; 0 means
 *   contiguous); weight int8 [N, K/size]; quant_buffer int32 [M, N] (required when size > 1).
 * reduce_mode 0 (exact, default): int32 partial accumulators are summed across ranks BEFORE the
 *   dequant epilogue, so the result is bit-identical to the unsharded linear; every rank passes
 *   the full-row scale_M and the same bias.
 * reduce_mode 1 (reference order): dequantize each partial to fp16, bias on rank 0 only, then fp16
 *   all-reduce (src/.../pmx/i8i8/row_parallel_linear.cu:84,131-158).
 * weight_layout: as for the column-parallel linear (COL32 input shard [M, K/size], legacy weight shard, operands
 *   re-laid out into `ws` of roundup(M*K/size, 256) + roundup(N*K/size, 256) bytes).
 */
int32_t pplb200_i8i8_row_parallel_linear(pplb200_stream_t stream, const void* input, int64_t M, int64_t input_ld,
                                         const void* weight, const void* optional_bias,
                                         const void* scale_M, const void* scale_N,
                                         float down_scale_M, float down_scale_N,
                                         int64_t in_features, int64_t out_features, int32_t weight_layout,
                                         int32_t rank, int32_t size, void* nccl_comm,
                                         int32_t input_is_parallel, int32_t reduce_mode, void* quant_buffer,
                                         void* ws, int64_t ws_bytes, void* output);

/*
 * Row-parallel linear over peer-mapped memory (ranks of one NVLink domain, one GPU per rank,
 * size <= 8).  Same result as pplb200_i8i8_row_parallel_linear with reduce_mode 0 -- bit-identical
 * to the unsharded linear -- but without a collective library on the data path: the GEMM stores
 * each raw int32 tile into the buffer of the rank that owns those output rows while it computes
 * the next tiles, the owner sums the `size` partials, applies scale and bias once, and the other
 * ranks fetch its finished fp16 rows.  Stands where the reference runs dequantize + fp16
 * all-reduce (src/ppl/kernel/llm/cuda/pmx/i8i8/row_parallel_linear.cu:113-160).
 *
 * Set-up, once per process and rank (these calls allocate and synchronise; the linear does not):
 *   pplb200_p2p_create        cudaMalloc of `bytes` (>= pplb200_i8i8_row_parallel_p2p_bytes of the
 *                             largest M, N used) on the current device, flags cleared.
 *   pplb200_p2p_export        64-byte inter-process handle of that buffer (host memory).
 *   pplb200_p2p_connect       maps the peers' buffers from the handles of all ranks (size x 64
 *                             bytes, rank order, exchanged by the caller); every rank must have
 *                             created its context before any rank's first linear call.
 *   pplb200_p2p_connect_local same, for contexts created in this process (one process driving
 *                             several devices): `peer_ctx` holds `size` context pointers.
 *
 * The linear: all ranks call it with the same M, N, K, in the same order on their contexts.
 * M % size == 0 (else RC_UNSUPPORTED: use the collective path), out_features % 8 == 0,
 * (in_features / size) % 16 == 0.  `input` is this rank's K shard [M, in_features / size] with
 * leading dimension input_ld (0: dense); scale_M are the full-row scales [M]; weight is the
 * shard [out_features, in_features / size]; output fp16 [M, out_features] is complete on every
 * rank when the call's work on `stream` has finished.
 * `phases`: 7 for the whole operation.  The bits (1 produce, 2 reduce, 4 gather) let one process
 * that drives several ranks on one stream enqueue the phases rank after rank.
 * With 7, large problems on four or more ranks are cut into two column chunks and the reduction and
 * row exchange of the first chunk run on a second stream (owned by the context) under the GEMM of the
 * second; 7 + 8 forces that schedule where the shape allows it, 7 + 16 forces the single-chunk one.
 * Waits on peers are bounded (about two seconds); pplb200_p2p_status returns a non-zero word
 * when one expired (bit 0: partial sums missing, bit 1: finished rows missing, bit 2: row maxima missing) -- the output of
 * that call is then undefined and later calls do not wait until the word is reset.
 */
int64_t pplb200_i8i8_row_parallel_p2p_bytes(int64_t M, int64_t out_features, int32_t size);
int32_t pplb200_p2p_create(int32_t rank, int32_t size, int64_t bytes, void** ctx_out);
int32_t pplb200_p2p_export(void* ctx, void* handle64_host);
int32_t pplb200_p2p_connect(void* ctx, const void* handles_host);
int32_t pplb200_p2p_connect_local(void* ctx, void* const* peer_ctx);
int32_t pplb200_p2p_destroy(void* ctx);
int32_t pplb200_p2p_status(void* ctx, int32_t reset);
int32_t pplb200_i8i8_row_parallel_linear_p2p(pplb200_stream_t stream, void* ctx, const void* input, int64_t M,
                                             int64_t input_ld, const void* weight, const void* optional_bias,
                                             const void* scale_M, const void* scale_N,
                                             float down_scale_M, float down_scale_N,
                                             int64_t in_features, int64_t out_features,
                                             int32_t phases, void* output);

/*
 * Column-parallel linear with gather_output over peer-mapped memory: what the reference does with dequantize ->
 * ncclAllGather -> [size, M, N/size] -> [M, N] transpose (src/ppl/kernel/llm/cuda/pmx/i8i8/column_parallel_linear.cu:86-89,159-179),
 * done by the GEMM's epilogue itself: every finished fp16 tile of this rank's [M, N/size] block is stored straight
 * into the gathered [M, N] matrix of EVERY rank, at column offset rank * N/size, in whole 128-byte lines, while the
 * following tiles are computed; a flag per rank then says "my block is in your area", and each rank copies the
 * gathered matrix from its peer-mapped area into `output`.  No collective library, no transpose pass.
 * `ctx` is a connected context of pplb200_p2p_create whose buffer holds at least
 * pplb200_i8i8_row_parallel_p2p_bytes(M, out_features, size) bytes (the gathered matrix lives where the row-parallel
 * operator keeps its partial sums: give the two operators separate contexts, or put a stream-level barrier across
 * the ranks between them).  input int8 [M, in_features] (replicated), weight int8 [out_features / size, in_features],
 * scale_N / bias this rank's slices, scale_M [M]; output fp16 [M, out_features], identical on every rank and
 * bit-identical to the unsharded linear.  (out_features / size) % 8 == 0, in_features % 16 == 0.
 * phases: 3 for the operation; 1 = compute and deliver, 2 = wait for the peers and copy out (lets one process that
 * drives several ranks on one stream run "1" for every rank, then "2" for every rank).  A rank does not overwrite a
 * peer's area before that peer has copied the previous result out (bounded wait; bits 3 and 4 of
 * pplb200_p2p_status report a missing block / a peer that never consumed).
 */
int32_t pplb200_i8i8_column_parallel_linear_p2p(pplb200_stream_t stream, void* ctx, const void* input, int64_t M,
                                                const void* weight, const void* optional_bias, const void* scale_M,
                                                const void* scale_N, float down_scale_M, float down_scale_N,
                                                int64_t in_features, int64_t out_features, int32_t phases, void* output);

/*
 * Per-token quantizer for activations that are sharded along the quantized dimension (the input
 * of a row-parallel linear as the preceding column-parallel operator leaves it): every rank passes
 * its shard [batch, shard_dim] fp16, dense.  The row scale comes from the maximum over the WHOLE
 * row: the ranks exchange their shard maxima through the peer-mapped buffer of `ctx` inside the
 * kernel, so int8 values and scales equal those of pplb200_i8i8_minmax_quantize_fp16 on the
 * unsharded rows (src/ppl/kernel/llm/cuda/pmx/i8i8/quantize.cu:27-124), bit for bit, while each
 * rank reads only its shard, once.  `scale` [batch] is the full-row scale on every rank.
 * batch <= 16384, shard_dim % 16 == 0, shard_dim <= 32768; all ranks call it with the same batch,
 * in the same order on their contexts.  phases: 3 for the operation; 1 only publishes the shard
 * maxima (lets one process that drives several ranks on one stream run "1" for every rank and then
 * "3" for every rank; a "1" must be followed by a "3" on the SAME input before anything else is quantized on the
 * context: it publishes under the tag of the operation that the "3" completes).  The kernel is launched
 * cooperatively (the whole grid resident at once, or the launch fails): keep the device free enough for it.
 * A wait that expires sets bit 2 of pplb200_p2p_status.
 */
int32_t pplb200_i8i8_minmax_quantize_fp16_p2p(pplb200_stream_t stream, void* ctx, const void* input, int64_t batch,
                                              int64_t shard_dim, float up_scale, int32_t phases,
                                              void* q, void* scale);

/*
 * NCCL plumbing for callers that do not already own a communicator (tests, bench).
 * unique id: 128 bytes, host memory.  Not part of the reference surface (ppl.nn.llm creates
 * its communicators itself and hands them over in ppl::common::NcclParam).
 */
int32_t pplb200_nccl_get_unique_id(void* id128_host);
int32_t pplb200_nccl_comm_init(const void* id128_host, int32_t rank, int32_t size, void** comm_out);
int32_t pplb200_nccl_comm_destroy(void* comm);

/*
 * Device-side health word of the GEMM kernel: every bounded wait in the kernel that gives
 * up records a code here instead of hanging.  Returns 0 if no kernel launched on the current
 * device has timed out since the last call with reset != 0.  Reads the word as it is now on a private
 * stream (no other stream is waited for): synchronise the streams you launched on before asking about them.
 */
int32_t pplb200_i8i8_gemm_status(int32_t reset);

/*
 * Diagnostics (process-wide switch, not thread-safe, off by default): with a non-NULL device array of
 * 8 x uint64 per CTA (296 CTAs at most), later launches of the CTA-pair GEMM record per CTA the SM cycles
 * [0] the MMA thread ran, [1] it waited for operand tiles, [2] it waited for a free accumulator,
 * [3] the TMA thread waited for a free slot, [4] the TMA thread ran, [5] the first epilogue warp waited for
 * an accumulator, [6] that warp ran.  NULL switches the recording off again.
 */
void pplb200_debug_gemm_stall_counters(void* counters);

/*
 * Diagnostics (process-wide switch, not thread-safe, on by default): when few 256 x 256 output tiles are left over
 * after the full waves of one tile per CTA pair, the CTA-pair GEMM cuts them along K into slices that different pairs
 * compute at once and sums the slices in the workspace (integer sums: the result does not depend on it).
 * enabled = 0 computes every tile on one pair, 1 (the default) lets the launcher weigh the K blocks saved against the
 * cost of the exchange, 2 slices whenever the shape and the workspace allow it; for A/B timing.
 */
void pplb200_debug_gemm_tail_split(int32_t enabled);

/*
 * Storage-order change of a [rows, cols] matrix of int8 (elem_bytes 1) or int32 (elem_bytes 4) elements between
 * any two of ROW_MAJOR, COL32, COL32_2R_4R4 and COL4_4R2_8C (index maps of
 * include/ppl/kernel/llm/cuda/common/matrix_layout.h:34-142; no counterpart function in the reference, whose
 * callers prepare such weights offline).  Meant for load time: weights stored for the Turing / Ampere kernels
 * -> ROW_MAJOR once, instead of on every call of a linear.  src != dst; cols % 32 == 0 when a tiled order is
 * involved (cols % 4 otherwise); rows % 32 == 0 for COL32_2R_4R4, rows % 8 == 0 for COL4_4R2_8C.
 */
int32_t pplb200_i8i8_relayout(pplb200_stream_t stream, const void* src, int32_t src_layout, void* dst, int32_t dst_layout,
                              int64_t rows, int64_t cols, int32_t elem_bytes);

/*
 * Measurement probes (no counterpart in the reference; they give the roofline denominators that
 * bench.py reports against).  `result24` is a 24-byte device record the launch fills:
 *   uint64 cycles, uint64 nanoseconds (of CTA 0, from first issue to completion), uint32 status, uint32 pad;
 * status != 0 means a bounded wait inside the probe gave up.
 * tensor_peak: every SM issues `mmas_per_cta` back-to-back tcgen05.mma kind::i8 (M 128 x N x K 32 per CTA, or
 *   M 256 x N x K 32 per CTA pair) on operands resident in shared memory.  shape: bit 0 = CTA pairs, bit 1 = rotate
 *   over four accumulator tiles (N <= 64), bits 8 and up = N (0 means 256).  With
 *   stream_src != NULL every CTA also keeps bulk copies from that buffer (stream_bytes, >= 32 KiB) into spare
 *   shared memory in flight, one 32 KiB copy per four MMAs -- the fill rate of a GEMM main loop -- so the figure
 *   becomes the ceiling with the copy engine competing for shared memory.  commit_pattern: bits 0-7 = issue a
 *   tcgen05.commit after every that many MMAs (0: only at the end), bit 8 = plus one to the partner CTA,
 *   bit 9 = one multicast commit to both CTAs instead: what releasing operand slots costs the issue stream.
 * stream_read: one launch reads `bytes` (a multiple of 32 KiB is used) from `src` with bulk asynchronous copies
 *   and discards them; the record's two uint64 then hold the global-timer nanoseconds of the earliest CTA start
 *   and of the latest CTA end (the launch as the device saw it, without the host's enqueue latency).
 */
int32_t pplb200_probe_tensor_peak(pplb200_stream_t stream, int32_t shape, int32_t mmas_per_cta, int32_t commit_pattern,
                                  const void* stream_src,
                                  int64_t stream_bytes, void* result24);
int32_t pplb200_probe_stream_read(pplb200_stream_t stream, const void* src, int64_t bytes, void* result24);

/*
 * Host-only helper: element offset of (row, col) in a [rows, cols] matrix stored in `layout`
 * (the index maps of include/ppl/kernel/llm/cuda/common/matrix_layout.h:34-142); -1 for an
 * unknown layout.
 */
int64_t pplb200_layout_offset(int32_t layout, int64_t rows, int64_t cols, int64_t row, int64_t col);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif
#endif
