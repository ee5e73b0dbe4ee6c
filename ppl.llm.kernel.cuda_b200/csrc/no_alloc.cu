// Allocation-free variant of the int8 GEMM with fused dequant + per-token re-quantize.
//
// The regular entry point (pplb200_i8i8_gemm, epilogue mode 2) needs a few bytes of scratch per
// token row -- the running maximum |y| of the row, combined across CTAs with atomicMax -- and takes
// them from a caller-supplied workspace.  Some callers have no way to come up with device memory at
// the moment they need this op: an inference runtime that handed every byte of HBM to its own
// arena / KV-cache pool at start-up and forbids cudaMalloc afterwards; code running inside a region
// where the CUDA allocation calls are illegal or synchronise the whole device (they serialise
// against all streams); plugins called through an interface that gives them tensors but no
// allocator.  For them the scratch lives here, in a fixed array that is part of the loaded module.
//
// Consequences the caller must know:
//   * the array has room for PPLB200_STATIC_SCRATCH_MAX_ROWS token rows (64 KiB); larger M is refused;
//   * every GPU that loads this library holds the array until the process exits;
//   * all calls on a device share it, and it keeps whatever the previous call left: this entry
//     point clears the part it uses (stream-ordered, before the GEMM), and two calls whose GPU work
//     overlaps (different streams) race on it -- keep calls on one stream, or order them;
//   * the first call on each device looks up the array's device address (one-time set-up); make
//     that first call before any stream capture begins.
#include "common.cuh"
#include "../../include/pplb200_i8i8.h"

#include <mutex>

namespace {

constexpr int64_t kMaxRows = PPLB200_STATIC_SCRATCH_MAX_ROWS;

// Per-row maximum |y| as float bits.  In host code this name is only a handle for the runtime: it
// is NOT a device address and must never be handed to a kernel; the address comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) uint32_t g_row_absmax_scratch[kMaxRows];

std::mutex g_mutex;
uint32_t* g_scratch_ptr[64] = {};

// Device address of the scratch array on the CURRENT device; resolved once per device.
uint32_t* scratch_on_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        uint32_t* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_row_absmax_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            pplb200::fail(pplb200::RC_DEVICE_RUNTIME_ERROR, "cudaGetSymbolAddress(scratch) failed: %s", cudaGetErrorString(e));
            return nullptr;
        }
        g_scratch_ptr[dev] = ptr;
    }
    return g_scratch_ptr[dev];
}

} // namespace

using namespace pplb200;

extern "C" int32_t pplb200_i8i8_gemm_requant_static_scratch(
    pplb200_stream_t stream_, const void* A, int64_t lda, const void* B, int64_t ldb, int64_t M, int64_t N, int64_t K,
    const void* scale_M, const void* scale_N, const void* optional_bias, float down_scale_M, float down_scale_N,
    float requant_up_scale, void* out, void* out_q, void* out_q_scale) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (M < 0 || N < 0 || K <= 0) return fail(RC_INVALID_VALUE, "bad GEMM extents M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
    if (M > kMaxRows)
        return fail(RC_INVALID_VALUE, "M=%lld exceeds the built-in scratch (%lld rows); use pplb200_i8i8_gemm with a workspace",
                    (long long)M, (long long)kMaxRows);
    if (M == 0 || N == 0) return RC_SUCCESS;
    if (!A || !B || !out || !out_q || !out_q_scale || !scale_M || !scale_N) return fail(RC_INVALID_VALUE, "null pointer");
    if (K % 16 || lda % 16 || ldb % 16 || lda < K || ldb < K) return fail(RC_INVALID_VALUE, "K, lda, ldb must be multiples of 16 and lda, ldb >= K");
    if (N % 16) return fail(RC_INVALID_VALUE, "N must be a multiple of 16, got %lld", (long long)N);
    if (!aligned16(A) || !aligned16(B) || !aligned16(out) || !aligned16(out_q) || !aligned16(scale_N) ||
        (optional_bias && !aligned16(optional_bias)))
        return fail(RC_INVALID_VALUE, "A, B, out, out_q, scale_N and bias must be 16-byte aligned");

    uint32_t* scratch = scratch_on_current_device();
    if (scratch == nullptr) return RC_DEVICE_RUNTIME_ERROR;

    // The row maxima must start at zero and the array still holds the previous call's values.
    if (cudaMemsetAsync(scratch, 0, (size_t)M * sizeof(uint32_t), stream) != cudaSuccess)
        return fail(RC_DEVICE_RUNTIME_ERROR, "clearing the scratch failed: %s", cudaGetErrorString(cudaGetLastError()));

    GemmArgs g;
    g.A = (const int8_t*)A; g.lda = lda; g.B = (const int8_t*)B; g.ldb = ldb;
    g.M = M; g.N = N; g.K = K; g.mode = EPI_DEQUANT_F16_REQUANT_I8;
    g.scale_m = (const half*)scale_M; g.scale_n = (const half*)scale_N; g.bias = (const half*)optional_bias;
    g.down_m = down_scale_M; g.down_n = down_scale_N;
    g.out = out; g.ldc = N;
    g.row_absmax_bits = scratch;
    g.pdl = false;
    int32_t rc = launch_gemm(stream, g);
    if (rc != RC_SUCCESS) return rc;
    return launch_quantize(stream, (const half*)out, M, N, requant_up_scale, LAYOUT_ROW_MAJOR, (int8_t*)out_q,
                           (half*)out_q_scale, scratch, nullptr, false);
}
