// TEST INFRASTRUCTURE ONLY.  C entry points around the reference's own,
// unmodified i8i8 operators (compiled from the reference tree next to this
// file by oracle/Makefile) so that tests and the bench can run them on the GPU
// as the parity comparator and as the "reference arm" of the benchmark.
#include "ppl/kernel/llm/cuda/pmx/i8i8/quantize.h"
#include "ppl/kernel/llm/cuda/pmx/i8i8/column_parallel_linear.h"
#include "ppl/kernel/llm/cuda/pmx/i8i8/row_parallel_linear.h"
#include "ppl/kernel/llm/cuda/cublas/gemm.h"
#include "cudakernel/memory/transpose.h"

#include <cublasLt.h>
#include <mutex>
#include <nccl.h>
#include <string.h>

namespace refns = ppl::kernel::llm::cuda;

// ---- the transpose the column-parallel linear needs (gather_output && size > 1)
template <typename T>
__global__ void refshim_transpose01(const T* in, int64_t d0, int64_t d1, int64_t d2, T* out) {
    int64_t total = d0 * d1 * d2;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t c = i % d2, b = (i / d2) % d1, a = i / (d2 * d1);
        out[(b * d0 + a) * d2 + c] = in[i];
    }
}

ppl::common::RetCode PPLCUDATranspose01ForwardImp(
    cudaStream_t stream, const void* input, ppl::common::datatype_t dtype,
    int64_t dim0, int64_t dim1, int64_t dim2, void* output) {
    if (ppl::common::GetSizeOfDataType(dtype) != 2) return ppl::common::RC_UNSUPPORTED;
    refshim_transpose01<uint16_t><<<1024, 256, 0, stream>>>((const uint16_t*)input, dim0, dim1, dim2, (uint16_t*)output);
    return ppl::common::RC_SUCCESS;
}

namespace {
struct RefState {
    cublasLtHandle_t lt = nullptr;
    refns::cublas::AlgoCache cache;
};
RefState& state() {
    static RefState s;
    static std::once_flag once;
    std::call_once(once, [] { cublasLtCreate(&s.lt); });
    return s;
}
}

extern "C" {

int32_t ref_minmax_quantize_fp16(cudaStream_t stream, const void* in, int64_t batch, int64_t dim, float up_scale,
                                 int32_t layout, void* q, void* scale) {
    return (int32_t)refns::pmx::i8i8::minmax_quantize_fp16(stream, in, batch, dim, up_scale,
                                                           (refns::matrix_layout_t)layout, q, scale);
}

int32_t ref_minmax_dequantize_fp16(cudaStream_t stream, const void* acc, const void* bias, const void* sm,
                                   const void* sn, int64_t batch, int64_t dim, float down_m, float down_n,
                                   int32_t layout, void* out) {
    return (int32_t)refns::pmx::i8i8::minmax_dequantize_fp16(stream, acc, bias, sm, sn, batch, dim, down_m, down_n,
                                                             (refns::matrix_layout_t)layout, out);
}

int32_t ref_skip_rmsnorm_minmax_quantize_fp16(cudaStream_t stream, const void* in, const void* weight, const void* skip,
                                              float eps, int64_t batch, int64_t dim, float up_scale, int32_t layout,
                                              void* skip_out, void* out_scale, void* out) {
    return (int32_t)refns::pmx::i8i8::skip_rmsnorm_minmax_quantize_fp16(stream, in, weight, skip, eps, batch, dim, up_scale,
                                                                        (refns::matrix_layout_t)layout, skip_out, out_scale, out);
}

int32_t ref_minmax_dequantize_split3_fp16(cudaStream_t stream, const void* in, const void* bias, const void* sb, const void* sc,
                                          int64_t batch, int64_t dim, int64_t d0, int64_t d1, int64_t d2, float down_b,
                                          float down_c, int32_t layout, void* o0, void* o1, void* o2) {
    return (int32_t)refns::pmx::i8i8::minmax_dequantize_split3_fp16(stream, in, bias, sb, sc, batch, dim, d0, d1, d2, down_b, down_c,
                                                                    (refns::matrix_layout_t)layout, o0, o1, o2);
}

int32_t ref_minmax_requantize_silu_fp16(cudaStream_t stream, const void* in, const void* sb, const void* sc, const void* gate,
                                        const void* gsb, const void* gsc, int64_t batch, int64_t dim, int32_t layout,
                                        float up, float down_b, float down_c, void* ws, void* out, void* scale) {
    return (int32_t)refns::pmx::i8i8::minmax_requantize_silu_fp16(stream, in, sb, sc, gate, gsb, gsc, batch, dim,
                                                                  (refns::matrix_layout_t)layout, up, down_b, down_c, ws, out, scale);
}

int32_t ref_minmax_requantize_swiglu_fp16(cudaStream_t stream, const void* in, const void* sb, const void* sc, int64_t batch,
                                          int64_t dim, float beta, int32_t layout, float up, float down_b, float down_c,
                                          void* ws, void* out, void* scale) {
    return (int32_t)refns::pmx::i8i8::minmax_requantize_swiglu_fp16(stream, in, sb, sc, batch, dim, beta,
                                                                    (refns::matrix_layout_t)layout, up, down_b, down_c, ws, out, scale);
}

// C[M,N] i32 = A[M,K] i8 * B[N,K]^T i8 through the reference's cuBLASLt wrapper
// (first call per shape bucket runs its autotuner, which synchronises the host).
int32_t ref_gemm_i8i8i32(cudaStream_t stream, const void* A, const void* B, int64_t M, int64_t N, int64_t K,
                         void* workspace, int64_t workspace_bytes, void* C) {
    RefState& s = state();
    return (int32_t)refns::cublas::gemm_i8i8i32(stream, s.lt, nullptr, false, K, ppl::common::DATATYPE_INT8, A,
                                                true, K, ppl::common::DATATYPE_INT8, B, nullptr, M, N, K, 1, 0,
                                                workspace_bytes, workspace, &s.cache, N,
                                                ppl::common::DATATYPE_INT32, C);
}

// The reference's column_parallel_linear on one rank (size 1), ROW_MAJOR weights.
// gather_output != 0: int32 GEMM result in quant_buffer, fp16 in out.  == 0: raw int32 in out.
int32_t ref_column_parallel_linear(cudaStream_t stream, const void* xq, const void* w, const void* bias,
                                   const void* sm, const void* sn, float down_m, float down_n,
                                   int64_t M, int64_t N, int64_t K, int32_t gather_output, void* quant_buffer,
                                   void* workspace, int64_t workspace_bytes, void* out) {
    RefState& s = state();
    ppl::common::TensorShape in_shape(ppl::common::DATATYPE_INT8, {M, K});
    ppl::common::TensorShape w_shape(ppl::common::DATATYPE_INT8, {N, K});
    ppl::common::TensorShape b_shape(ppl::common::DATATYPE_FLOAT16, {N});
    ppl::common::TensorShape o_shape(gather_output ? ppl::common::DATATYPE_FLOAT16 : ppl::common::DATATYPE_INT32, {M, N});
    ppl::common::NcclParam nccl;
    return (int32_t)refns::pmx::i8i8::column_parallel_linear(
        stream, s.lt, nullptr, &in_shape, xq, &w_shape, w, &b_shape, bias, sm, sn, down_m, down_n, K, N,
        refns::MATRIX_LAYOUT_ROW_MAJOR, &nccl, gather_output != 0, nullptr, quant_buffer, workspace_bytes, workspace,
        &s.cache, &o_shape, out);
}

// The reference's row_parallel_linear on one rank of `size` (comm may be null when size == 1).
int32_t ref_row_parallel_linear(cudaStream_t stream, const void* xq, const void* w, const void* bias,
                                const void* sm, const void* sn, float down_m, float down_n,
                                int64_t M, int64_t N, int64_t K_total, int32_t rank, int32_t size, void* comm,
                                void* quant_buffer, void* workspace, int64_t workspace_bytes, void* out) {
    RefState& s = state();
    ppl::common::TensorShape in_shape(ppl::common::DATATYPE_INT8, {M, K_total / size});
    ppl::common::TensorShape w_shape(ppl::common::DATATYPE_INT8, {N, K_total / size});
    ppl::common::TensorShape b_shape(ppl::common::DATATYPE_FLOAT16, {N});
    ppl::common::TensorShape o_shape(ppl::common::DATATYPE_FLOAT16, {M, N});
    ppl::common::NcclParam nccl;
    nccl.rank = rank; nccl.size = size; nccl.comm = (ncclComm_t)comm;
    return (int32_t)refns::pmx::i8i8::row_parallel_linear(
        stream, s.lt, nullptr, &in_shape, xq, &w_shape, w, &b_shape, bias, sm, sn, down_m, down_n, K_total, N,
        refns::MATRIX_LAYOUT_ROW_MAJOR, &nccl, true, nullptr, quant_buffer, workspace_bytes, workspace,
        &s.cache, &o_shape, out);
}

// The reference's column_parallel_linear on one rank of `size` with gather_output = true: dequantized
// shard -> gather_buffer -> all-gather -> [size, M, N/size] -> [M, N] transpose into `out`.
int32_t ref_column_parallel_linear_tp(cudaStream_t stream, const void* xq, const void* w, const void* bias,
                                      const void* sm, const void* sn, float down_m, float down_n,
                                      int64_t M, int64_t N_total, int64_t K, int32_t rank, int32_t size, void* comm,
                                      void* gather_buffer, void* quant_buffer, void* workspace, int64_t workspace_bytes,
                                      void* out) {
    RefState& s = state();
    ppl::common::TensorShape in_shape(ppl::common::DATATYPE_INT8, {M, K});
    ppl::common::TensorShape w_shape(ppl::common::DATATYPE_INT8, {N_total / size, K});
    ppl::common::TensorShape b_shape(ppl::common::DATATYPE_FLOAT16, {N_total / size});
    ppl::common::TensorShape o_shape(ppl::common::DATATYPE_FLOAT16, {M, N_total});
    ppl::common::NcclParam nccl;
    nccl.rank = rank; nccl.size = size; nccl.comm = (ncclComm_t)comm;
    return (int32_t)refns::pmx::i8i8::column_parallel_linear(
        stream, s.lt, nullptr, &in_shape, xq, &w_shape, w, &b_shape, bias, sm, sn, down_m, down_n, K, N_total,
        refns::MATRIX_LAYOUT_ROW_MAJOR, &nccl, true, gather_buffer, quant_buffer, workspace_bytes, workspace,
        &s.cache, &o_shape, out);
}

// The reference's GEMM on the Turing / Ampere operand orders (A, C in COL32; B in COL32_2R_4R4 or
// COL4_4R2_8C).  Returns the reference's RetCode; *cublas_status_out receives nothing more than that
// (the wrapper folds the cuBLASLt status into RC_DEVICE_RUNTIME_ERROR and logs it).
int32_t ref_gemm_i8i8i32_col32(cudaStream_t stream, const void* input_col32, const void* kernel, int64_t M, int64_t N,
                               int64_t K, int32_t use_4r4_kernel, void* output_col32) {
    RefState& s = state();
    return (int32_t)refns::cublas::gemm_i8i8i32_col32(stream, s.lt, input_col32, kernel, M, N, K, use_4r4_kernel != 0,
                                                      output_col32);
}

// Communicator plumbing for the reference arm of the benchmark and the multi-GPU parity tests, so
// that they need nothing but this library (same NCCL as the collectives above).
int32_t ref_nccl_get_unique_id(void* id128_host) {
    static_assert(sizeof(ncclUniqueId) == 128, "unique id size");
    return ncclGetUniqueId((ncclUniqueId*)id128_host) == ncclSuccess ? 0 : 10;
}
int32_t ref_nccl_comm_init(const void* id128_host, int32_t rank, int32_t size, void** comm_out) {
    ncclUniqueId id;
    memcpy(&id, id128_host, sizeof(id));
    ncclComm_t comm = nullptr;
    if (ncclCommInitRank(&comm, size, id, rank) != ncclSuccess) return 10;
    *comm_out = comm;
    return 0;
}
int32_t ref_nccl_comm_destroy(void* comm) { return comm && ncclCommDestroy((ncclComm_t)comm) != ncclSuccess ? 10 : 0; }

}
