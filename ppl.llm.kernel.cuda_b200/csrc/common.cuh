// Shared declarations of the sm_100a i8i8 linear library: return codes, error
// recording, small device helpers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace pplb200 {

// Numeric values of ppl::common::RetCode that this path returns.
enum : int32_t {
    RC_SUCCESS = 0,
    RC_UNSUPPORTED = 2,
    RC_INVALID_VALUE = 4,
    RC_DEVICE_RUNTIME_ERROR = 10,
};

// matrix_layout_t numbering of the reference (common/matrix_layout.h:25-31).
enum : int32_t {
    LAYOUT_ROW_MAJOR = 0,
    LAYOUT_COL_MAJOR = 1,
    LAYOUT_COL32 = 2,
    LAYOUT_COL32_2R_4R4 = 3,
    LAYOUT_COL4_4R2_8C = 4,
};

enum : int32_t {
    EPI_RAW_I32 = 0,
    EPI_DEQUANT_F16 = 1,
    EPI_DEQUANT_F16_REQUANT_I8 = 2,
    EPI_SWIGLU_F16 = 3, // internal: fused gate+up projection, see pplb200_i8i8_gate_up_swiglu_requant
    EPI_PUSH_I32 = 4,   // internal: raw int32 tiles stored into the row owner's peer-mapped buffer
    EPI_GATHER_F16 = 5, // internal: dequantized fp16 tiles stored into EVERY rank's peer-mapped [M, N_total] area
};

constexpr int kMaxPeers = 8;

// Records a message retrievable through pplb200_last_error() and returns `rc`.
int32_t fail(int32_t rc, const char* fmt, ...);
void clear_error();

// Checks the launch status of the kernel just enqueued.
int32_t check_launch(const char* what);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// (row, col) -> element offset in each of the reference's five layouts.
__host__ __device__ inline int64_t layout_offset(int32_t layout, int64_t rows, int64_t cols, int64_t r, int64_t c) {
    (void)cols;
    switch (layout) {
    case LAYOUT_ROW_MAJOR: return r * cols + c;
    case LAYOUT_COL_MAJOR: return c * rows + r;
    case LAYOUT_COL32: return ((c >> 5) * rows + r) * 32 + (c & 31);
    case LAYOUT_COL32_2R_4R4: {
        const int64_t rt = r & 31;
        const int64_t slot = ((((rt & 7) >> 1) << 2) + (rt >> 3)) * 2 + (rt & 1); // 32-row interleave
        return (c >> 5) * rows * 32 + (r >> 5) * 1024 + slot * 32 + (c & 31);
    }
    default: { // LAYOUT_COL4_4R2_8C
        const int64_t cc = c & 31;
        const int64_t line = (r & ~int64_t(7)) + ((r & 1) << 2) + (cc >> 3);
        const int64_t quad = ((cc & 4) ? 4 : 0) + ((r & 7) >> 1);
        return (c >> 5) * rows * 32 + line * 32 + quad * 4 + (cc & 3);
    }
    }
}

// ---- kernels / launchers implemented across the translation units ----

// given_absmax_bits != null: rows are quantized with that precomputed max |x| (float bits) instead of
// scanning the row.  zero_absmax_bits != null: the kernel also clears that per-row array (for the
// GEMM that follows).  pdl: launch as a programmatic dependent of the preceding kernel in the stream.
int32_t launch_quantize(cudaStream_t stream, const half* in, int64_t batch, int64_t dim, float up_scale,
                        int32_t layout, int8_t* q, half* scale, const uint32_t* given_absmax_bits,
                        uint32_t* zero_absmax_bits = nullptr, bool pdl = false);

int32_t launch_dequantize(cudaStream_t stream, const int32_t* acc, const half* bias, const half* scale_m,
                          const half* scale_n, int64_t batch, int64_t dim, float down_m, float down_n,
                          int32_t layout, half* out);

int32_t launch_skip_rmsnorm_quantize(cudaStream_t stream, const half* input, const half* weight, const half* skip,
                                     float eps, int64_t batch, int64_t dim, float up_scale, int32_t layout,
                                     half* skip_out, half* scale_out, int8_t* q);

// consumers of the raw int32 accumulators (activation_requant.cu)
int32_t act_silu(cudaStream_t stream, const void* input, const void* sb, const void* sc, const void* gate, const void* gsb,
                 const void* gsc, int64_t batch, int64_t dim, int32_t layout, float up, float down_b, float down_c,
                 void* workspace, void* out, void* scale_out, bool requant);
int32_t act_swiglu(cudaStream_t stream, const void* input, const void* sb, const void* sc, int64_t batch, int64_t dim,
                   float beta, int32_t layout, float up, float down_b, float down_c, void* workspace, void* out,
                   void* scale_out);
int32_t dequantize_split3(cudaStream_t stream, const void* acc, const void* bias, const void* sm, const void* sn,
                          int64_t batch, int64_t dim, int64_t d0, int64_t d1, int64_t d2, float down_m, float down_n,
                          int32_t layout, void* o0, void* o1, void* o2);

// storage-order change of a [rows, cols] matrix of 1- or 4-byte elements between any two of ROW_MAJOR, COL32,
// COL32_2R_4R4, COL4_4R2_8C (cols % 4 == 0 and the layouts' own divisibility rules checked by the caller)
int32_t launch_relayout(cudaStream_t stream, const void* src, int32_t src_layout, void* dst, int32_t dst_layout,
                        int64_t rows, int64_t cols, int32_t elem_bytes);

int32_t launch_transpose01_f16(cudaStream_t stream, const half* in, int64_t d0, int64_t d1, int64_t d2, half* out);

struct GemmArgs {
    const int8_t* A; int64_t lda;
    const int8_t* B; int64_t ldb;
    int64_t M, N, K;
    int32_t mode;
    const half* scale_m; const half* scale_n; const half* bias;
    float down_m, down_n;
    void* out; int64_t ldc;
    uint32_t* row_absmax_bits; // mode 2: per-row max |y| as float bits, zeroed by the launcher
    bool pdl = false;          // launch as a programmatic dependent of the preceding kernel
    float beta = 1.0f;         // EPI_SWIGLU_F16
    // EPI_RAW_I32 only: out = raw_alpha * acc + raw_beta * out + raw_bias[n] in wrapping int32 (the scaling and
    // int32 bias of the reference's gemm_i8i8i32, src/ppl/kernel/llm/cuda/cublas/gemm.cu:187-188,239-243)
    int32_t raw_alpha = 1, raw_beta = 0;
    const int32_t* raw_bias = nullptr;
    // EPI_PUSH_I32: output row r belongs to rank r / push_rows; it is stored at
    // push_base[owner] + ((push_rank * push_rows + r % push_rows) * ldc + col) (int32 elements).
    int32_t* push_base[kMaxPeers] = {};
    int32_t push_rows = 0, push_rank = 0;
    // EPI_GATHER_F16: the tile's fp16 values go to ((half*)push_base[d]) + row * ldc + gather_col0 + col for every
    // rank d < gather_ranks (ldc = width of the gathered output)
    int32_t gather_ranks = 0;
    int64_t gather_col0 = 0;
    // Optional scratch (256-byte aligned, kSkWsBytes, contents arbitrary) that lets the CTA-pair kernel cut the few
    // tiles left over after its full waves along K and compute the slices on different pairs at once; without it every
    // tile is computed by one pair.  Two launches that may run at the same time need separate scratches.
    void* sk_ws = nullptr;
    int64_t sk_ws_bytes = 0;
};
// at most kSkMaxTiles leftover tiles (half the CTA pairs of a 148-SM device) of 256 x 256 int32 partial sums,
// preceded by the warps' arrival counters
constexpr int64_t kSkMaxTiles = 40;
constexpr int64_t kSkTileBytes = 256 * 256 * 4;
constexpr int64_t kSkStateBytes = 2048;
constexpr int64_t kSkWsBytes = kSkStateBytes + kSkMaxTiles * kSkTileBytes;
static_assert(kSkMaxTiles * 8 * 4 <= kSkStateBytes, "arrival counters");
int32_t launch_gemm_decode(cudaStream_t stream, const GemmArgs& a, unsigned int* status, bool pdl);
int32_t launch_gemm(cudaStream_t stream, const GemmArgs& a);
int32_t gemm_status(int32_t reset);
void set_stall_counters(void* dev_ptr);
void set_tail_split(int mode);
unsigned long long* stall_counters();

} // namespace pplb200
