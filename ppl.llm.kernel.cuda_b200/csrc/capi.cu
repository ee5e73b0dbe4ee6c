// extern "C" surface of the library (declared in include/pplb200_i8i8.h): argument checks,
// workspace carving and the launch sequences of the single-device path.
#include "common.cuh"
#include "../../include/pplb200_i8i8.h"

#include <mutex>
#include <stdarg.h>
#include <string.h>

namespace pplb200 {

namespace {
thread_local char g_err[512] = "";
}

int32_t fail(int32_t rc, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    fprintf(stderr, "[pplb200][ERROR] %s\n", g_err);
    return rc;
}
void clear_error() { g_err[0] = '\0'; }

int32_t check_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(RC_DEVICE_RUNTIME_ERROR, "%s launch failed: %s", what, cudaGetErrorString(e));
    return RC_SUCCESS;
}

namespace {

constexpr int64_t WS_ALIGN = 256;

// row maxima of the fused re-quantize
int64_t absmax_ws_bytes(int64_t M, int32_t mode) {
    return mode == EPI_DEQUANT_F16_REQUANT_I8 ? round_up(M * 4, WS_ALIGN) : 0;
}
// What the GEMM asks for: the row maxima, then (large batches only) the scratch through which CTA pairs share the
// tiles of the last waves.  The second part is optional at run time: with a smaller workspace every tile is computed
// by one pair.
int64_t gemm_ws_bytes(int64_t M, int32_t mode) {
    return absmax_ws_bytes(M, mode) + (M > 128 ? kSkWsBytes : 0);
}

int32_t check_gemm_args(const void* A, int64_t lda, const void* B, int64_t ldb, int64_t M, int64_t N, int64_t K,
                        int32_t mode, const void* scale_M, const void* scale_N, const void* bias, void* out,
                        int64_t ldc, void* out_q, void* out_q_scale) {
    if (M < 0 || N < 0 || K <= 0) return fail(RC_INVALID_VALUE, "bad GEMM extents M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
    if (mode < EPI_RAW_I32 || mode > EPI_DEQUANT_F16_REQUANT_I8) return fail(RC_UNSUPPORTED, "unknown epilogue mode %d", mode);
    if (M == 0 || N == 0) return RC_SUCCESS;
    if (!A || !B || !out) return fail(RC_INVALID_VALUE, "null A/B/out");
    if (K % 16 || lda % 16 || ldb % 16) return fail(RC_INVALID_VALUE, "K, lda, ldb must be multiples of 16 (K=%lld lda=%lld ldb=%lld)", (long long)K, (long long)lda, (long long)ldb);
    if (lda < K || ldb < K || ldc < N) return fail(RC_INVALID_VALUE, "leading dimension smaller than the row length");
    if (N % 8) return fail(RC_INVALID_VALUE, "N must be a multiple of 8, got %lld", (long long)N);
    if (!aligned16(A) || !aligned16(B) || !aligned16(out)) return fail(RC_INVALID_VALUE, "A, B and out must be 16-byte aligned");
    const int64_t out_elem = mode == EPI_RAW_I32 ? 4 : 2;
    if ((ldc * out_elem) % 16) return fail(RC_INVALID_VALUE, "ldc must keep rows 16-byte aligned");
    if (mode != EPI_RAW_I32) {
        if (!scale_M || !scale_N) return fail(RC_INVALID_VALUE, "dequant epilogue needs scale_M and scale_N");
        if (!aligned16(scale_N) || (bias && !aligned16(bias))) return fail(RC_INVALID_VALUE, "scale_N / bias must be 16-byte aligned");
    }
    if (mode == EPI_DEQUANT_F16_REQUANT_I8) {
        if (!out_q || !out_q_scale) return fail(RC_INVALID_VALUE, "re-quantize epilogue needs out_q and out_q_scale");
        if (N % 16 || ldc != N || !aligned16(out_q)) return fail(RC_INVALID_VALUE, "re-quantize epilogue needs N %% 16 == 0, ldc == N, aligned out_q");
    }
    return RC_SUCCESS;
}

} // namespace

// chained: the caller has just enqueued the activation quantizer on `stream`, which also cleared the
// row-maximum scratch; the GEMM and the re-quantizer are then launched as programmatic dependents.
int32_t gemm_entry(cudaStream_t stream, const void* A, int64_t lda, const void* B, int64_t ldb, int64_t M, int64_t N,
                   int64_t K, int32_t mode, const void* scale_M, const void* scale_N, const void* bias, float down_M,
                   float down_N, float requant_up, void* ws, int64_t ws_bytes, void* out, int64_t ldc, void* out_q,
                   void* out_q_scale, bool chained) {
    int32_t rc = check_gemm_args(A, lda, B, ldb, M, N, K, mode, scale_M, scale_N, bias, out, ldc, out_q, out_q_scale);
    if (rc != RC_SUCCESS || M == 0 || N == 0) return rc;
    GemmArgs g;
    g.A = (const int8_t*)A; g.lda = lda; g.B = (const int8_t*)B; g.ldb = ldb;
    g.M = M; g.N = N; g.K = K; g.mode = mode;
    g.scale_m = (const half*)scale_M; g.scale_n = (const half*)scale_N; g.bias = (const half*)bias;
    g.down_m = down_M; g.down_n = down_N;
    g.out = out; g.ldc = ldc;
    g.row_absmax_bits = nullptr;
    const int64_t need = absmax_ws_bytes(M, mode);
    if (mode == EPI_DEQUANT_F16_REQUANT_I8) {
        if (!ws || ws_bytes < need) return fail(RC_INVALID_VALUE, "workspace too small: %lld < %lld", (long long)ws_bytes, (long long)need);
        g.row_absmax_bits = (uint32_t*)ws;
        if (!chained && cudaMemsetAsync(ws, 0, (size_t)M * 4, stream) != cudaSuccess)
            return fail(RC_DEVICE_RUNTIME_ERROR, "memset failed");
    }
    if (ws && ws_bytes > need) {
        g.sk_ws = (char*)ws + need;
        g.sk_ws_bytes = ws_bytes - need;
    }
    g.pdl = chained;
    rc = launch_gemm(stream, g);
    if (rc != RC_SUCCESS) return rc;
    if (mode == EPI_DEQUANT_F16_REQUANT_I8)
        rc = launch_quantize(stream, (const half*)out, M, N, requant_up, LAYOUT_ROW_MAJOR, (int8_t*)out_q,
                             (half*)out_q_scale, g.row_absmax_bits, nullptr, /*pdl=*/M <= 128);
    return rc;
}

} // namespace pplb200

using namespace pplb200;

extern "C" {

const char* pplb200_version(void) { return "pplb200 i8i8 0.1 sm_100a"; }
const char* pplb200_last_error(void) { return g_err; }

int32_t pplb200_i8i8_minmax_quantize_fp16(pplb200_stream_t stream, const void* in, int64_t batch, int64_t quant_dim,
                                          float up_scale, int32_t to_layout, void* q, void* scale) {
    if (to_layout != LAYOUT_ROW_MAJOR && to_layout != LAYOUT_COL32 && to_layout != LAYOUT_COL32_2R_4R4)
        return fail(RC_UNSUPPORTED, "unsupported matrix layout: %d", to_layout);
    if (batch < 0 || quant_dim < 0) return fail(RC_INVALID_VALUE, "negative extent");
    if (batch == 0 || quant_dim == 0) return RC_SUCCESS;
    if (quant_dim % 16) return fail(RC_INVALID_VALUE, "quant_dim must be a multiple of 16, got %lld", (long long)quant_dim);
    if (to_layout != LAYOUT_ROW_MAJOR && quant_dim % 32) return fail(RC_INVALID_VALUE, "COL32 layouts need quant_dim %% 32 == 0");
    if (to_layout == LAYOUT_COL32_2R_4R4 && batch % 32) return fail(RC_INVALID_VALUE, "COL32_2R_4R4 needs batch %% 32 == 0");
    if (!in || !q || !scale) return fail(RC_INVALID_VALUE, "null pointer");
    if (!aligned16(in) || !aligned16(q)) return fail(RC_INVALID_VALUE, "in and q must be 16-byte aligned");
    if (batch > 0x7fffffffLL) return fail(RC_UNSUPPORTED, "batch beyond 2^31 - 1");
    return launch_quantize((cudaStream_t)stream, (const half*)in, batch, quant_dim, up_scale, to_layout, (int8_t*)q,
                           (half*)scale, nullptr);
}

int32_t pplb200_i8i8_minmax_dequantize_fp16(pplb200_stream_t stream, const void* acc, const void* optional_bias,
                                            const void* scale_per_batch, const void* scale_per_channel,
                                            int64_t batch, int64_t quant_dim, float down_scale_batch,
                                            float down_scale_channel, int32_t from_layout, void* out) {
    if (quant_dim % 4 != 0) return fail(RC_INVALID_VALUE, "channel must be aligned with 4, but channel = %lld", (long long)quant_dim);
    if (from_layout < LAYOUT_ROW_MAJOR || from_layout > LAYOUT_COL4_4R2_8C) return fail(RC_UNSUPPORTED, "unsupported matrix layout: %d", from_layout);
    if (batch < 0 || quant_dim < 0) return fail(RC_INVALID_VALUE, "negative extent");
    if (batch == 0 || quant_dim == 0) return RC_SUCCESS;
    if (!acc || !scale_per_batch || !scale_per_channel || !out) return fail(RC_INVALID_VALUE, "null pointer");
    return launch_dequantize((cudaStream_t)stream, (const int32_t*)acc, (const half*)optional_bias,
                             (const half*)scale_per_batch, (const half*)scale_per_channel, batch, quant_dim,
                             down_scale_batch, down_scale_channel, from_layout, (half*)out);
}

int32_t pplb200_i8i8_skip_rmsnorm_minmax_quantize_fp16(pplb200_stream_t stream, const void* input, const void* weight,
                                                       const void* optional_skip, float eps, int64_t batch,
                                                       int64_t normalize_shape, float up_scale, int32_t to_layout,
                                                       void* skip_out, void* output_scale, void* output) {
    if (to_layout != LAYOUT_ROW_MAJOR && to_layout != LAYOUT_COL32 && to_layout != LAYOUT_COL32_2R_4R4)
        return fail(RC_UNSUPPORTED, "unsupported matrix layout: %d", to_layout);
    if (batch < 0 || normalize_shape < 0) return fail(RC_INVALID_VALUE, "negative extent");
    if (batch == 0 || normalize_shape == 0) return RC_SUCCESS;
    if (normalize_shape % 16) return fail(RC_INVALID_VALUE, "normalize_shape must be a multiple of 16, got %lld", (long long)normalize_shape);
    if (to_layout != LAYOUT_ROW_MAJOR && normalize_shape % 32) return fail(RC_INVALID_VALUE, "COL32 layouts need normalize_shape %% 32 == 0");
    if (to_layout == LAYOUT_COL32_2R_4R4 && batch % 32) return fail(RC_INVALID_VALUE, "COL32_2R_4R4 needs batch %% 32 == 0");
    if (!input || !weight || !skip_out || !output_scale || !output) return fail(RC_INVALID_VALUE, "null pointer");
    if (!aligned16(input) || !aligned16(weight) || !aligned16(skip_out) || !aligned16(output) ||
        (optional_skip && !aligned16(optional_skip)))
        return fail(RC_INVALID_VALUE, "input, weight, skip, skip_out and output must be 16-byte aligned");
    if (batch > 0x7fffffffLL) return fail(RC_UNSUPPORTED, "batch beyond 2^31 - 1");
    return launch_skip_rmsnorm_quantize((cudaStream_t)stream, (const half*)input, (const half*)weight, (const half*)optional_skip,
                                        eps, batch, normalize_shape, up_scale, to_layout, (half*)skip_out,
                                        (half*)output_scale, (int8_t*)output);
}

int32_t pplb200_i8i8_minmax_dequantize_split3_fp16(pplb200_stream_t stream, const void* input, const void* optional_bias,
                                                   const void* scale_per_batch, const void* scale_per_channel,
                                                   int64_t batch, int64_t quant_dim, int64_t split_dim_0,
                                                   int64_t split_dim_1, int64_t split_dim_2, float down_scale_batch,
                                                   float down_scale_channel, int32_t from_layout, void* output_0,
                                                   void* output_1, void* output_2) {
    return dequantize_split3((cudaStream_t)stream, input, optional_bias, scale_per_batch, scale_per_channel, batch, quant_dim,
                             split_dim_0, split_dim_1, split_dim_2, down_scale_batch, down_scale_channel, from_layout,
                             output_0, output_1, output_2);
}

int32_t pplb200_i8i8_minmax_dequantize_silu_fp16(pplb200_stream_t stream, const void* input, const void* input_scale_per_batch,
                                                 const void* input_scale_per_channel, const void* optional_gate,
                                                 const void* gate_scale_per_batch, const void* gate_scale_per_channel,
                                                 int64_t batch, int64_t quant_dim, int32_t from_layout,
                                                 float down_scale_batch, float down_scale_channel, void* output) {
    return act_silu((cudaStream_t)stream, input, input_scale_per_batch, input_scale_per_channel, optional_gate,
                    gate_scale_per_batch, gate_scale_per_channel, batch, quant_dim, from_layout, 0.0f, down_scale_batch,
                    down_scale_channel, nullptr, output, nullptr, false);
}

int32_t pplb200_i8i8_minmax_requantize_silu_fp16(pplb200_stream_t stream, const void* input, const void* input_scale_per_batch,
                                                 const void* input_scale_per_channel, const void* optional_gate,
                                                 const void* gate_scale_per_batch, const void* gate_scale_per_channel,
                                                 int64_t batch, int64_t quant_dim, int32_t layout, float up_scale,
                                                 float down_scale_batch, float down_scale_channel, void* workspace,
                                                 void* output, void* scale) {
    return act_silu((cudaStream_t)stream, input, input_scale_per_batch, input_scale_per_channel, optional_gate,
                    gate_scale_per_batch, gate_scale_per_channel, batch, quant_dim, layout, up_scale, down_scale_batch,
                    down_scale_channel, workspace, output, scale, true);
}

int32_t pplb200_i8i8_minmax_requantize_swiglu_fp16(pplb200_stream_t stream, const void* input, const void* input_scale_per_batch,
                                                   const void* input_scale_per_channel, int64_t batch, int64_t quant_dim,
                                                   float beta, int32_t layout, float up_scale, float down_scale_batch,
                                                   float down_scale_channel, void* workspace, void* output, void* scale) {
    return act_swiglu((cudaStream_t)stream, input, input_scale_per_batch, input_scale_per_channel, batch, quant_dim, beta, layout,
                      up_scale, down_scale_batch, down_scale_channel, workspace, output, scale);
}

namespace {
// The fused form needs the CTA-pair kernel: enough 256-row x 128-channel tiles for every pair, and
// the x / gate halves of the weight matrix aligned to the 128-row tiles.
bool swiglu_fusable(int64_t M, int64_t D) { return M > 128 && D % 128 == 0 && ((M + 255) / 256) * (D / 128) >= 74; }
}

int64_t pplb200_i8i8_gate_up_swiglu_workspace_bytes(int64_t M, int64_t act_dim, int64_t K) {
    (void)K;
    const int64_t maxima = round_up(M * 4 + 4, WS_ALIGN);
    return swiglu_fusable(M, act_dim) ? maxima : maxima + round_up(M * 2 * act_dim * 4, WS_ALIGN);
}

int32_t pplb200_i8i8_gate_up_swiglu_requant(pplb200_stream_t stream_, const void* input, int64_t lda, const void* weight,
                                            int64_t M, int64_t act_dim, int64_t K, const void* scale_M,
                                            const void* scale_N, float beta, float up_scale, float down_scale_M,
                                            float down_scale_N, void* ws, int64_t ws_bytes, void* activated,
                                            void* out_q, void* out_q_scale) {
    cudaStream_t stream = (cudaStream_t)stream_;
    const int64_t D = act_dim;
    if (M < 0 || D < 0 || K <= 0) return fail(RC_INVALID_VALUE, "bad extents");
    if (M == 0 || D == 0) return RC_SUCCESS;
    if (K % 16 || lda % 16 || lda < K || D % 16) return fail(RC_INVALID_VALUE, "K, lda, act_dim must be multiples of 16 and lda >= K");
    if (!input || !weight || !scale_M || !scale_N || !activated || !out_q || !out_q_scale) return fail(RC_INVALID_VALUE, "null pointer");
    if (!aligned16(input) || !aligned16(weight) || !aligned16(scale_N) || !aligned16(activated) || !aligned16(out_q))
        return fail(RC_INVALID_VALUE, "operands must be 16-byte aligned");
    const int64_t need = pplb200_i8i8_gate_up_swiglu_workspace_bytes(M, D, K);
    if (!ws || ws_bytes < need) return fail(RC_INVALID_VALUE, "workspace too small: %lld < %lld", (long long)ws_bytes, (long long)need);
    if ((reinterpret_cast<uintptr_t>(ws) & (WS_ALIGN - 1)) != 0) return fail(RC_INVALID_VALUE, "workspace must be 256-byte aligned");
    uint32_t* maxima = (uint32_t*)ws;

    if (!swiglu_fusable(M, D)) {
        // small problems: raw int32 GEMM, then the stand-alone SwiGLU + re-quantize kernel
        void* acc = (char*)ws + round_up(M * 4 + 4, WS_ALIGN);
        int32_t rc = gemm_entry(stream, input, lda, weight, K, M, 2 * D, K, EPI_RAW_I32, nullptr, nullptr, nullptr, 0.f, 0.f, 0.f,
                                nullptr, 0, acc, 2 * D, nullptr, nullptr, false);
        if (rc != RC_SUCCESS) return rc;
        return act_swiglu(stream, acc, scale_M, scale_N, M, D, beta, LAYOUT_ROW_MAJOR, up_scale, down_scale_M, down_scale_N,
                          activated, out_q, out_q_scale);
    }

    if (cudaMemsetAsync(maxima, 0, (size_t)M * 4, stream) != cudaSuccess) return fail(RC_DEVICE_RUNTIME_ERROR, "memset failed");
    GemmArgs g;
    g.A = (const int8_t*)input; g.lda = lda; g.B = (const int8_t*)weight; g.ldb = K;
    g.M = M; g.N = 2 * D; g.K = K; g.mode = EPI_SWIGLU_F16;
    g.scale_m = (const half*)scale_M; g.scale_n = (const half*)scale_N; g.bias = nullptr;
    g.down_m = down_scale_M; g.down_n = down_scale_N;
    g.out = activated; g.ldc = D;
    g.row_absmax_bits = maxima;
    g.beta = beta;
    int32_t rc = launch_gemm(stream, g);
    if (rc != RC_SUCCESS) return rc;
    return launch_quantize(stream, (const half*)activated, M, D, up_scale, LAYOUT_ROW_MAJOR, (int8_t*)out_q, (half*)out_q_scale,
                           maxima, nullptr, false);
}

int64_t pplb200_i8i8_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t epilogue_mode) {
    (void)N; (void)K;
    return gemm_ws_bytes(M, epilogue_mode);
}

int32_t pplb200_i8i8_gemm(pplb200_stream_t stream, const void* A, int64_t lda, const void* B, int64_t ldb,
                          int64_t M, int64_t N, int64_t K, int32_t epilogue_mode,
                          const void* scale_M, const void* scale_N, const void* optional_bias,
                          float down_scale_M, float down_scale_N, float requant_up_scale,
                          void* ws, int64_t ws_bytes, void* out, int64_t ldc, void* out_q, void* out_q_scale) {
    return gemm_entry((cudaStream_t)stream, A, lda, B, ldb, M, N, K, epilogue_mode, scale_M, scale_N, optional_bias,
                      down_scale_M, down_scale_N, requant_up_scale, ws, ws_bytes, out, ldc, out_q, out_q_scale, false);
}

int32_t pplb200_i8i8_gemm_i32(pplb200_stream_t stream, const void* A, int64_t lda, const void* B, int64_t ldb,
                              int64_t M, int64_t N, int64_t K, int32_t alpha, int32_t beta, const void* optional_bias_i32,
                              void* C, int64_t ldc) {
    int32_t rc = check_gemm_args(A, lda, B, ldb, M, N, K, EPI_RAW_I32, nullptr, nullptr, nullptr, C, ldc, nullptr, nullptr);
    if (rc != RC_SUCCESS || M == 0 || N == 0) return rc;
    if (optional_bias_i32 && !aligned16(optional_bias_i32)) return fail(RC_INVALID_VALUE, "int32 bias must be 16-byte aligned");
    GemmArgs g;
    g.A = (const int8_t*)A; g.lda = lda; g.B = (const int8_t*)B; g.ldb = ldb;
    g.M = M; g.N = N; g.K = K; g.mode = EPI_RAW_I32;
    g.scale_m = nullptr; g.scale_n = nullptr; g.bias = nullptr;
    g.down_m = 0.f; g.down_n = 0.f;
    g.out = C; g.ldc = ldc;
    g.row_absmax_bits = nullptr;
    g.raw_alpha = alpha; g.raw_beta = beta; g.raw_bias = (const int32_t*)optional_bias_i32;
    return launch_gemm((cudaStream_t)stream, g);
}

int64_t pplb200_i8i8_linear_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t epilogue_mode) {
    (void)N;
    return round_up(M * K, WS_ALIGN) + round_up(M * 2, WS_ALIGN) + gemm_ws_bytes(M, epilogue_mode);
}

int32_t pplb200_i8i8_linear_fp16(pplb200_stream_t stream, const void* x, const void* W, const void* scale_N,
                                 const void* optional_bias, int64_t M, int64_t N, int64_t K,
                                 float up_scale, float down_scale_M, float down_scale_N,
                                 int32_t epilogue_mode, float requant_up_scale,
                                 void* ws, int64_t ws_bytes, void* y, void* y_q, void* y_q_scale) {
    if (epilogue_mode != EPI_DEQUANT_F16 && epilogue_mode != EPI_DEQUANT_F16_REQUANT_I8)
        return fail(RC_UNSUPPORTED, "linear_fp16 epilogue must be DEQUANT_F16 or DEQUANT_F16_REQUANT_I8");
    if (M < 0 || N < 0 || K <= 0) return fail(RC_INVALID_VALUE, "bad extents");
    if (M == 0 || N == 0) return RC_SUCCESS;
    const int64_t need = pplb200_i8i8_linear_workspace_bytes(M, N, K, epilogue_mode);
    if (!ws || ws_bytes < need) return fail(RC_INVALID_VALUE, "workspace too small: %lld < %lld", (long long)ws_bytes, (long long)need);
    if ((reinterpret_cast<uintptr_t>(ws) & (WS_ALIGN - 1)) != 0) return fail(RC_INVALID_VALUE, "workspace must be 256-byte aligned");
    char* base = (char*)ws;
    void* xq = base;
    void* sm = base + round_up(M * K, WS_ALIGN);
    void* gws = base + round_up(M * K, WS_ALIGN) + round_up(M * 2, WS_ALIGN);
    if (K % 16) return fail(RC_INVALID_VALUE, "K must be a multiple of 16, got %lld", (long long)K);
    if (!x || !aligned16(x)) return fail(RC_INVALID_VALUE, "x must be a 16-byte aligned device pointer");
    if (M > 0x7fffffffLL) return fail(RC_UNSUPPORTED, "M beyond 2^31 - 1");
    // the quantizer also clears the row-maximum scratch of the fused re-quantize
    uint32_t* absmax = epilogue_mode == EPI_DEQUANT_F16_REQUANT_I8 ? (uint32_t*)gws : nullptr;
    // The quantizer itself is launched as a programmatic dependent of whatever precedes it on the stream: it
    // touches no memory before its griddepcontrol.wait, so this only hides its launch latency (back-to-back
    // calls of this function then overlap the tail of one call with the head of the next).
    int32_t rc = launch_quantize((cudaStream_t)stream, (const half*)x, M, K, up_scale, LAYOUT_ROW_MAJOR, (int8_t*)xq,
                                 (half*)sm, nullptr, absmax, /*pdl=*/M <= 128);
    if (rc != RC_SUCCESS) return rc;
    return gemm_entry((cudaStream_t)stream, xq, K, W, K, M, N, K, epilogue_mode, sm, scale_N, optional_bias, down_scale_M,
                      down_scale_N, requant_up_scale, gws, gemm_ws_bytes(M, epilogue_mode), y, N, y_q, y_q_scale, true);
}

int32_t pplb200_i8i8_relayout(pplb200_stream_t stream, const void* src, int32_t src_layout, void* dst, int32_t dst_layout,
                              int64_t rows, int64_t cols, int32_t elem_bytes) {
    auto known = [](int32_t l) { return l == LAYOUT_ROW_MAJOR || l == LAYOUT_COL32 || l == LAYOUT_COL32_2R_4R4 || l == LAYOUT_COL4_4R2_8C; };
    if (!known(src_layout) || !known(dst_layout)) return fail(RC_UNSUPPORTED, "unsupported matrix layout: %d -> %d", src_layout, dst_layout);
    if (elem_bytes != 1 && elem_bytes != 4) return fail(RC_UNSUPPORTED, "element size must be 1 (int8) or 4 (int32)");
    if (rows < 0 || cols < 0) return fail(RC_INVALID_VALUE, "negative extent");
    if (rows == 0 || cols == 0) return RC_SUCCESS;
    if (!src || !dst || src == dst) return fail(RC_INVALID_VALUE, "src / dst must be distinct non-null pointers");
    const bool tiled = src_layout != LAYOUT_ROW_MAJOR || dst_layout != LAYOUT_ROW_MAJOR;
    if (cols % 4 || (tiled && cols % 32)) return fail(RC_INVALID_VALUE, "cols must be a multiple of 32 for the tiled layouts (4 otherwise)");
    auto rows_ok = [&](int32_t l) { return l == LAYOUT_COL32_2R_4R4 ? rows % 32 == 0 : l == LAYOUT_COL4_4R2_8C ? rows % 8 == 0 : true; };
    if (!rows_ok(src_layout) || !rows_ok(dst_layout)) return fail(RC_INVALID_VALUE, "rows must be a multiple of 32 (COL32_2R_4R4) / 8 (COL4_4R2_8C)");
    if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & (elem_bytes == 1 ? 3 : 15))
        return fail(RC_INVALID_VALUE, "src / dst must be aligned to four elements");
    return launch_relayout((cudaStream_t)stream, src, src_layout, dst, dst_layout, rows, cols, elem_bytes);
}

// ---- host-buffer form of the fused linear ----------------------------------------------------
namespace {
struct HostPipe { // per device: two copy streams and the events that order them against the caller's stream
    bool ready = false;
    cudaStream_t in = nullptr, out = nullptr;
    cudaEvent_t start = nullptr, in_done[2] = {}, comp_done[2] = {}, out_done[2] = {};
};
HostPipe g_host_pipe[64];
std::mutex g_host_pipe_mutex; // one enqueue sequence at a time: the events of a device are shared by its callers

HostPipe* host_pipe() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    HostPipe& h = g_host_pipe[dev];
    if (!h.ready) {
        if (cudaStreamCreateWithFlags(&h.in, cudaStreamNonBlocking) != cudaSuccess ||
            cudaStreamCreateWithFlags(&h.out, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&h.start, cudaEventDisableTiming) != cudaSuccess)
            return nullptr;
        for (int i = 0; i < 2; ++i)
            if (cudaEventCreateWithFlags(&h.in_done[i], cudaEventDisableTiming) != cudaSuccess ||
                cudaEventCreateWithFlags(&h.comp_done[i], cudaEventDisableTiming) != cudaSuccess ||
                cudaEventCreateWithFlags(&h.out_done[i], cudaEventDisableTiming) != cudaSuccess)
                return nullptr;
        h.ready = true;
    }
    return &h;
}

int64_t host_chunk_rows(int64_t M, int64_t chunk_rows) {
    if (chunk_rows <= 0) chunk_rows = 1024;
    return chunk_rows < M ? chunk_rows : M;
}
} // namespace

int64_t pplb200_i8i8_linear_host_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t epilogue_mode, int64_t chunk_rows) {
    const int64_t c = host_chunk_rows(M, chunk_rows);
    const int64_t per_buf = round_up(c * K * 2, WS_ALIGN) + round_up(c * N * 2, WS_ALIGN) +
                            (epilogue_mode == EPI_DEQUANT_F16_REQUANT_I8 ? round_up(c * N, WS_ALIGN) + round_up(c * 2, WS_ALIGN) : 0) +
                            round_up(pplb200_i8i8_linear_workspace_bytes(c, N, K, epilogue_mode), WS_ALIGN);
    return 2 * per_buf;
}

int32_t pplb200_i8i8_linear_fp16_host(pplb200_stream_t stream_, const void* x_host, const void* W, const void* scale_N,
                                      const void* optional_bias, int64_t M, int64_t N, int64_t K, float up_scale,
                                      float down_scale_M, float down_scale_N, int32_t epilogue_mode, float requant_up_scale,
                                      int64_t chunk_rows, void* ws, int64_t ws_bytes, void* y_host, void* y_q_host,
                                      void* y_q_scale_host) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (epilogue_mode != EPI_DEQUANT_F16 && epilogue_mode != EPI_DEQUANT_F16_REQUANT_I8)
        return fail(RC_UNSUPPORTED, "linear_fp16_host epilogue must be DEQUANT_F16 or DEQUANT_F16_REQUANT_I8");
    if (M < 0 || N < 0 || K <= 0) return fail(RC_INVALID_VALUE, "bad extents");
    if (M == 0 || N == 0) return RC_SUCCESS;
    const bool requant = epilogue_mode == EPI_DEQUANT_F16_REQUANT_I8;
    if (!x_host || !y_host || (requant && (!y_q_host || !y_q_scale_host))) return fail(RC_INVALID_VALUE, "null host buffer");
    const int64_t need = pplb200_i8i8_linear_host_workspace_bytes(M, N, K, epilogue_mode, chunk_rows);
    if (!ws || ws_bytes < need) return fail(RC_INVALID_VALUE, "workspace too small: %lld < %lld", (long long)ws_bytes, (long long)need);
    if ((reinterpret_cast<uintptr_t>(ws) & (WS_ALIGN - 1)) != 0) return fail(RC_INVALID_VALUE, "workspace must be 256-byte aligned");
    std::lock_guard<std::mutex> lock(g_host_pipe_mutex);
    HostPipe* h = host_pipe();
    if (!h) return fail(RC_DEVICE_RUNTIME_ERROR, "stream / event set-up failed: %s", cudaGetErrorString(cudaGetLastError()));
    const int64_t c = host_chunk_rows(M, chunk_rows);
    const int64_t lin_ws = round_up(pplb200_i8i8_linear_workspace_bytes(c, N, K, epilogue_mode), WS_ALIGN);
    char* base = (char*)ws;
    char *xd[2], *yd[2], *yqd[2] = {nullptr, nullptr}, *ysd[2] = {nullptr, nullptr}, *lw[2];
    for (int b = 0; b < 2; ++b) {
        xd[b] = base; base += round_up(c * K * 2, WS_ALIGN);
        yd[b] = base; base += round_up(c * N * 2, WS_ALIGN);
        if (requant) { yqd[b] = base; base += round_up(c * N, WS_ALIGN); ysd[b] = base; base += round_up(c * 2, WS_ALIGN); }
        lw[b] = base; base += lin_ws;
    }
#define PPLB200_CU(call) do { if ((call) != cudaSuccess) return fail(RC_DEVICE_RUNTIME_ERROR, "%s failed: %s", #call, cudaGetErrorString(cudaGetLastError())); } while (0)
    // both copy streams start after whatever the caller has already enqueued on its stream
    PPLB200_CU(cudaEventRecord(h->start, stream));
    PPLB200_CU(cudaStreamWaitEvent(h->in, h->start, 0));
    PPLB200_CU(cudaStreamWaitEvent(h->out, h->start, 0));
    // Chunk sizes: the copy-out of the results is the longest of the three pipelines (PCIe, fp16 [rows, N]), and it can
    // only start once the first chunk has been copied in and computed.  So the first full chunk is fed in as c/8, c/8,
    // c/4, c/2 rows (each step's copy-in + compute still fits under the previous step's copy-out), which starts the
    // copy-out after an eighth of the fill time.
    const bool ramp = c >= 1024 && M >= 2 * c;
    int64_t chunk = 0, rows = 0;
    for (int64_t m0 = 0; m0 < M; m0 += rows, ++chunk) {
        const int b = (int)(chunk & 1);
        rows = !ramp || chunk >= 4 ? c : chunk < 2 ? c / 8 : chunk == 2 ? c / 4 : c / 2;
        if (rows > M - m0) rows = M - m0;
        // copy-in: the staging buffer is free once the linear of two chunks ago has read it
        if (chunk >= 2) PPLB200_CU(cudaStreamWaitEvent(h->in, h->comp_done[b], 0));
        PPLB200_CU(cudaMemcpyAsync(xd[b], (const char*)x_host + m0 * K * 2, (size_t)(rows * K * 2), cudaMemcpyHostToDevice, h->in));
        PPLB200_CU(cudaEventRecord(h->in_done[b], h->in));
        // compute on the caller's stream: needs the chunk's input, and its output buffers copied out (two chunks ago)
        PPLB200_CU(cudaStreamWaitEvent(stream, h->in_done[b], 0));
        if (chunk >= 2) PPLB200_CU(cudaStreamWaitEvent(stream, h->out_done[b], 0));
        const int32_t rc = pplb200_i8i8_linear_fp16(stream_, xd[b], W, scale_N, optional_bias, rows, N, K, up_scale, down_scale_M,
                                                    down_scale_N, epilogue_mode, requant_up_scale, lw[b], lin_ws, yd[b], yqd[b], ysd[b]);
        if (rc != RC_SUCCESS) return rc;
        PPLB200_CU(cudaEventRecord(h->comp_done[b], stream));
        // copy-out
        PPLB200_CU(cudaStreamWaitEvent(h->out, h->comp_done[b], 0));
        PPLB200_CU(cudaMemcpyAsync((char*)y_host + m0 * N * 2, yd[b], (size_t)(rows * N * 2), cudaMemcpyDeviceToHost, h->out));
        if (requant) {
            PPLB200_CU(cudaMemcpyAsync((char*)y_q_host + m0 * N, yqd[b], (size_t)(rows * N), cudaMemcpyDeviceToHost, h->out));
            PPLB200_CU(cudaMemcpyAsync((char*)y_q_scale_host + m0 * 2, ysd[b], (size_t)(rows * 2), cudaMemcpyDeviceToHost, h->out));
        }
        PPLB200_CU(cudaEventRecord(h->out_done[b], h->out));
    }
    // join: work enqueued on the caller's stream after this call sees the complete host result
    PPLB200_CU(cudaStreamWaitEvent(stream, h->out_done[0], 0));
    if (chunk >= 2) PPLB200_CU(cudaStreamWaitEvent(stream, h->out_done[1], 0));
#undef PPLB200_CU
    return RC_SUCCESS;
}

int32_t pplb200_i8i8_gemm_status(int32_t reset) { return gemm_status(reset); }
void pplb200_debug_gemm_stall_counters(void* counters) { set_stall_counters(counters); }
void pplb200_debug_gemm_tail_split(int32_t enabled) { set_tail_split(enabled < 0 ? 0 : enabled > 2 ? 2 : enabled); }

// Host helper for tests: the library's (row, col) -> offset map for a layout.
int64_t pplb200_layout_offset(int32_t layout, int64_t rows, int64_t cols, int64_t row, int64_t col) {
    if (layout < LAYOUT_ROW_MAJOR || layout > LAYOUT_COL4_4R2_8C) return -1;
    return layout_offset(layout, rows, cols, row, col);
}

}
