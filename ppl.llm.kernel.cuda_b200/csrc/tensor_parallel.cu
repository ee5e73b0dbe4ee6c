// Tensor-parallel i8i8 linears over NCCL (one process per GPU).
//   column parallel (N sharded): no communication unless the caller asks for the gathered output
//   row parallel    (K sharded): int32 partial accumulators are summed across ranks BEFORE the
//                                dequant epilogue, so the sharded result equals the unsharded one
//                                bit for bit (integer addition is associative).
// Reference: src/ppl/kernel/llm/cuda/pmx/i8i8/column_parallel_linear.cu:29-182,
//            src/ppl/kernel/llm/cuda/pmx/i8i8/row_parallel_linear.cu:28-162.
#include "common.cuh"
#include "../../include/pplb200_i8i8.h"

#include <dlfcn.h>
#include <mutex>
#include <nccl.h>
#include <string.h>

// NCCL is bound at first use instead of at link time: a process that already carries an NCCL
// (for instance the one bundled with its deep-learning framework) keeps using that single copy,
// whatever the import order; otherwise the system libnccl.so.2 is loaded.
namespace {
struct NcclApi {
    bool ok = false;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

const NcclApi& nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
#define PPLB200_BIND(field, name) api.field = reinterpret_cast<decltype(api.field)>(dlsym(h, name))
        PPLB200_BIND(GetUniqueId, "ncclGetUniqueId");
        PPLB200_BIND(CommInitRank, "ncclCommInitRank");
        PPLB200_BIND(CommDestroy, "ncclCommDestroy");
        PPLB200_BIND(AllReduce, "ncclAllReduce");
        PPLB200_BIND(AllGather, "ncclAllGather");
        PPLB200_BIND(ReduceScatter, "ncclReduceScatter");
        PPLB200_BIND(GetErrorString, "ncclGetErrorString");
#undef PPLB200_BIND
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.AllGather &&
                 api.ReduceScatter && api.GetErrorString;
    });
    return api;
}
}

namespace pplb200 {
int32_t gemm_entry(cudaStream_t stream, const void* A, int64_t lda, const void* B, int64_t ldb, int64_t M, int64_t N,
                   int64_t K, int32_t mode, const void* scale_M, const void* scale_N, const void* bias, float down_M,
                   float down_N, float requant_up, void* ws, int64_t ws_bytes, void* out, int64_t ldc, void* out_q,
                   void* out_q_scale, bool chained = false);
}

using namespace pplb200;

namespace {

int32_t nccl_fail(const char* what, ncclResult_t r) {
    return fail(RC_DEVICE_RUNTIME_ERROR, "%s failed: %s", what, nccl_api().ok ? nccl_api().GetErrorString(r) : "NCCL not loaded");
}
int32_t nccl_missing() { return fail(RC_DEVICE_RUNTIME_ERROR, "libnccl.so.2 could not be loaded"); }
bool weight_layout_known(int32_t l) {
    return l == LAYOUT_ROW_MAJOR || l == LAYOUT_COL4_4R2_8C || l == LAYOUT_COL32_2R_4R4;
}

// Operands in the Turing / Ampere tensor-core orders.  With such a weight layout the reference runs
// gemm_i8i8i32_col32 (src/ppl/kernel/llm/cuda/cublas/gemm.cu:365-488): the int8 input is COL32 [M, K], the
// weight COL32_2R_4R4 or COL4_4R2_8C [N, K], and the int32 product COL32 [M, N]
// (pmx/i8i8/column_parallel_linear.cu:66-75,120-131).  The tensor cores of sm_100a read none of these orders, so
// both operands are re-laid out into the caller's workspace (row-major) first; a caller that can should convert
// its weights ONCE with pplb200_i8i8_relayout at load time and pass ROW_MAJOR instead.
struct LegacyOperands {
    const void* input;
    const void* weight;
    void* raw_tmp; // row-major int32 [M, N] scratch for the gather_output = false form
};

int64_t legacy_ws_bytes(int64_t M, int64_t N, int64_t K, bool want_raw) {
    return round_up(M * K, 256) + round_up(N * K, 256) + (want_raw ? round_up(M * N * 4, 256) : 0);
}

int32_t prepare_legacy(cudaStream_t stream, const void* input, const void* weight, int32_t weight_layout, int64_t M, int64_t N,
                       int64_t K, bool want_raw, void* ws, int64_t ws_bytes, LegacyOperands* out) {
    if (K % 32 || N % 32) return fail(RC_INVALID_VALUE, "COL32 operand orders need in_features %% 32 == 0 and out_features / size %% 32 == 0");
    const int64_t need = legacy_ws_bytes(M, N, K, want_raw);
    if (!ws || ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 255))
        return fail(RC_UNSUPPORTED, "weight layout %d needs a 256-byte aligned workspace of %lld bytes to re-lay the operands out "
                    "(got %lld); or convert the weights once with pplb200_i8i8_relayout and pass ROW_MAJOR",
                    weight_layout, (long long)need, (long long)ws_bytes);
    char* base = (char*)ws;
    void* a_rm = base;
    void* w_rm = base + round_up(M * K, 256);
    int32_t rc = launch_relayout(stream, input, LAYOUT_COL32, a_rm, LAYOUT_ROW_MAJOR, M, K, 1);
    if (rc != RC_SUCCESS) return rc;
    rc = launch_relayout(stream, weight, weight_layout, w_rm, LAYOUT_ROW_MAJOR, N, K, 1);
    if (rc != RC_SUCCESS) return rc;
    out->input = a_rm; out->weight = w_rm;
    out->raw_tmp = want_raw ? base + round_up(M * K, 256) + round_up(N * K, 256) : nullptr;
    return RC_SUCCESS;
}
}

extern "C" {

int32_t pplb200_i8i8_column_parallel_linear(pplb200_stream_t stream_, const void* input, int64_t M,
                                            const void* weight, const void* optional_bias,
                                            const void* scale_M, const void* scale_N,
                                            float down_scale_M, float down_scale_N,
                                            int64_t in_features, int64_t out_features, int32_t weight_layout,
                                            int32_t rank, int32_t size, void* nccl_comm,
                                            int32_t gather_output, void* gather_buffer, void* quant_buffer,
                                            void* ws, int64_t ws_bytes, void* output) {
    (void)quant_buffer;
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!weight_layout_known(weight_layout)) return fail(RC_UNSUPPORTED, "unsupported weight layout:%d", weight_layout);
    if (size < 1 || rank < 0 || rank >= size) return fail(RC_INVALID_VALUE, "bad rank/size %d/%d", rank, size);
    if (out_features % size) return fail(RC_INVALID_VALUE, "out_features %% size != 0");
    const int64_t Nw = out_features / size, K = in_features;

    LegacyOperands legacy = {};
    if (weight_layout != LAYOUT_ROW_MAJOR) {
        int32_t rc = prepare_legacy(stream, input, weight, weight_layout, M, Nw, K, !gather_output, ws, ws_bytes, &legacy);
        if (rc != RC_SUCCESS) return rc;
        input = legacy.input;
        weight = legacy.weight;
        ws = nullptr; ws_bytes = 0; // taken by the re-laid operands
    }

    if (!gather_output) { // raw int32 accumulators, no dequant (column_parallel_linear.cu:81-85,136)
        if (legacy.raw_tmp == nullptr)
            return gemm_entry(stream, input, K, weight, K, M, Nw, K, EPI_RAW_I32, nullptr, nullptr, nullptr, 0.f, 0.f, 0.f,
                              ws, ws_bytes, output, Nw, nullptr, nullptr);
        // legacy orders: the reference leaves the product in COL32
        int32_t rc = gemm_entry(stream, input, K, weight, K, M, Nw, K, EPI_RAW_I32, nullptr, nullptr, nullptr, 0.f, 0.f, 0.f,
                                nullptr, 0, legacy.raw_tmp, Nw, nullptr, nullptr);
        if (rc != RC_SUCCESS) return rc;
        return launch_relayout(stream, legacy.raw_tmp, LAYOUT_ROW_MAJOR, output, LAYOUT_COL32, M, Nw, 4);
    }

    if (size == 1)
        return gemm_entry(stream, input, K, weight, K, M, Nw, K, EPI_DEQUANT_F16, scale_M, scale_N, optional_bias,
                          down_scale_M, down_scale_N, 0.f, ws, ws_bytes, output, Nw, nullptr, nullptr);

    if (!gather_buffer || !nccl_comm) return fail(RC_INVALID_VALUE, "gather_output with size > 1 needs gather_buffer and a communicator");
    if (!nccl_api().ok) return nccl_missing();
    half* mine = (half*)gather_buffer + (int64_t)rank * M * Nw;
    int32_t rc = gemm_entry(stream, input, K, weight, K, M, Nw, K, EPI_DEQUANT_F16, scale_M, scale_N, optional_bias,
                            down_scale_M, down_scale_N, 0.f, ws, ws_bytes, mine, Nw, nullptr, nullptr);
    if (rc != RC_SUCCESS) return rc;
    ncclResult_t r = nccl_api().AllGather(mine, gather_buffer, (size_t)(M * Nw), ncclHalf, (ncclComm_t)nccl_comm, stream);
    if (r != ncclSuccess) return nccl_fail("ncclAllGather", r);
    return launch_transpose01_f16(stream, (const half*)gather_buffer, size, M, Nw, (half*)output);
}

int32_t pplb200_i8i8_row_parallel_linear(pplb200_stream_t stream_, const void* input, int64_t M, int64_t input_ld,
                                         const void* weight, const void* optional_bias,
                                         const void* scale_M, const void* scale_N,
                                         float down_scale_M, float down_scale_N,
                                         int64_t in_features, int64_t out_features, int32_t weight_layout,
                                         int32_t rank, int32_t size, void* nccl_comm,
                                         int32_t input_is_parallel, int32_t reduce_mode, void* quant_buffer,
                                         void* ws, int64_t ws_bytes, void* output) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!input_is_parallel) return fail(RC_UNSUPPORTED, "currently only support parallel input");
    if (!weight_layout_known(weight_layout)) return fail(RC_UNSUPPORTED, "unsupported weight layout:%d", weight_layout);
    if (size < 1 || rank < 0 || rank >= size) return fail(RC_INVALID_VALUE, "bad rank/size %d/%d", rank, size);
    if (in_features % size) return fail(RC_INVALID_VALUE, "in_features %% size != 0");
    if (reduce_mode != 0 && reduce_mode != 1) return fail(RC_INVALID_VALUE, "reduce_mode must be 0 or 1");
    const int64_t N = out_features, Kw = in_features / size;
    int64_t lda = input_ld > 0 ? input_ld : Kw;
    if (weight_layout != LAYOUT_ROW_MAJOR) { // COL32 input shard, legacy weight shard: see prepare_legacy
        if (input_ld > 0 && input_ld != Kw) return fail(RC_INVALID_VALUE, "a COL32 input has no leading dimension");
        LegacyOperands legacy = {};
        int32_t rc = prepare_legacy(stream, input, weight, weight_layout, M, N, Kw, false, ws, ws_bytes, &legacy);
        if (rc != RC_SUCCESS) return rc;
        input = legacy.input;
        weight = legacy.weight;
        lda = Kw;
        ws = nullptr; ws_bytes = 0; // taken by the re-laid operands
    }

    if (size == 1)
        return gemm_entry(stream, input, lda, weight, Kw, M, N, Kw, EPI_DEQUANT_F16, scale_M, scale_N, optional_bias,
                          down_scale_M, down_scale_N, 0.f, ws, ws_bytes, output, N, nullptr, nullptr);
    if (!nccl_comm) return fail(RC_INVALID_VALUE, "size > 1 needs a communicator");
    if (!nccl_api().ok) return nccl_missing();
    if (M == 0 || N == 0) return RC_SUCCESS;

    if (reduce_mode == 1) {
        // reference order: dequantize the partial (bias on rank 0 only), then sum in fp16
        const void* reduce_bias = rank == 0 ? optional_bias : nullptr;
        int32_t rc = gemm_entry(stream, input, lda, weight, Kw, M, N, Kw, EPI_DEQUANT_F16, scale_M, scale_N, reduce_bias,
                                down_scale_M, down_scale_N, 0.f, ws, ws_bytes, output, N, nullptr, nullptr);
        if (rc != RC_SUCCESS) return rc;
        ncclResult_t r = nccl_api().AllReduce(output, output, (size_t)(M * N), ncclHalf, ncclSum, (ncclComm_t)nccl_comm, stream);
        return r == ncclSuccess ? RC_SUCCESS : nccl_fail("ncclAllReduce(fp16)", r);
    }

    if (!quant_buffer) return fail(RC_INVALID_VALUE, "exact row-parallel reduction needs quant_buffer (int32 [M, N])");

    // Preferred schedule: the int32 partials are reduce-scattered over the ranks (each rank receives
    // the exact sums of its row slice), the slice is dequantized once, and the fp16 slices are
    // all-gathered -- 25 % less wire traffic than an int32 all-reduce and the epilogue work is split
    // over the ranks.  Everything is enqueued on the caller's stream: the library owns no stream or
    // event on this path, so concurrent callers on one device cannot disturb each other and the
    // sequence can be captured like any other stream work.  (A row-chunked form with the collectives
    // of chunk c on a second stream under the GEMM of chunk c + 1 measured slower on 2, 4 and 8
    // GPUs -- a persistent GEMM leaves the collectives' kernels no SMs -- and was removed.)
    if (M % size == 0) {
        const int64_t Ms = M / size; // rows per rank slice
        int32_t* acc = (int32_t*)quant_buffer;
        half* out16 = (half*)output;
        int32_t rc = gemm_entry(stream, input, lda, weight, Kw, M, N, Kw, EPI_RAW_I32, nullptr, nullptr, nullptr, 0.f, 0.f,
                                0.f, ws, ws_bytes, acc, N, nullptr, nullptr);
        if (rc != RC_SUCCESS) return rc;
        int32_t* mine = acc + (int64_t)rank * Ms * N; // reduce-scatter in place: this rank's slice
        ncclResult_t r = nccl_api().ReduceScatter(acc, mine, (size_t)(Ms * N), ncclInt32, ncclSum, (ncclComm_t)nccl_comm, stream);
        if (r != ncclSuccess) return nccl_fail("ncclReduceScatter(int32)", r);
        const int64_t row0 = (int64_t)rank * Ms;
        rc = launch_dequantize(stream, mine, (const half*)optional_bias, (const half*)scale_M + row0, (const half*)scale_N,
                               Ms, N, down_scale_M, down_scale_N, LAYOUT_ROW_MAJOR, out16 + row0 * N);
        if (rc != RC_SUCCESS) return rc;
        r = nccl_api().AllGather(out16 + row0 * N, out16, (size_t)(Ms * N), ncclHalf, (ncclComm_t)nccl_comm, stream);
        return r == ncclSuccess ? RC_SUCCESS : nccl_fail("ncclAllGather(fp16)", r);
    }

    // Fallback (M not divisible by the number of ranks): int32 all-reduce, then the epilogue on every rank.
    int32_t rc = gemm_entry(stream, input, lda, weight, Kw, M, N, Kw, EPI_RAW_I32, nullptr, nullptr, nullptr, 0.f, 0.f, 0.f,
                            ws, ws_bytes, quant_buffer, N, nullptr, nullptr);
    if (rc != RC_SUCCESS) return rc;
    ncclResult_t r = nccl_api().AllReduce(quant_buffer, quant_buffer, (size_t)(M * N), ncclInt32, ncclSum, (ncclComm_t)nccl_comm, stream);
    if (r != ncclSuccess) return nccl_fail("ncclAllReduce(int32)", r);
    return launch_dequantize(stream, (const int32_t*)quant_buffer, (const half*)optional_bias, (const half*)scale_M,
                             (const half*)scale_N, M, N, down_scale_M, down_scale_N, LAYOUT_ROW_MAJOR, (half*)output);
}

int32_t pplb200_nccl_get_unique_id(void* id128_host) {
    static_assert(sizeof(ncclUniqueId) == 128, "unique id size");
    if (!nccl_api().ok) return nccl_missing();
    ncclResult_t r = nccl_api().GetUniqueId((ncclUniqueId*)id128_host);
    return r == ncclSuccess ? RC_SUCCESS : nccl_fail("ncclGetUniqueId", r);
}

int32_t pplb200_nccl_comm_init(const void* id128_host, int32_t rank, int32_t size, void** comm_out) {
    if (!nccl_api().ok) return nccl_missing();
    ncclUniqueId id;
    memcpy(&id, id128_host, sizeof(id));
    ncclComm_t comm = nullptr;
    ncclResult_t r = nccl_api().CommInitRank(&comm, size, id, rank);
    if (r != ncclSuccess) return nccl_fail("ncclCommInitRank", r);
    *comm_out = comm;
    return RC_SUCCESS;
}

int32_t pplb200_nccl_comm_destroy(void* comm) {
    if (!comm) return RC_SUCCESS;
    if (!nccl_api().ok) return nccl_missing();
    ncclResult_t r = nccl_api().CommDestroy((ncclComm_t)comm);
    return r == ncclSuccess ? RC_SUCCESS : nccl_fail("ncclCommDestroy", r);
}

}
