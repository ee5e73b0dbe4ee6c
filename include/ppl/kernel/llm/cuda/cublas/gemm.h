// int8 GEMM entry point with the reference's signature
// (include/ppl/kernel/llm/cuda/cublas/gemm.h:56-90), forwarded to the sm_100a tcgen05 kernel
// through the C ABI.  cuBLASLt handle, algorithm, algorithm cache and cuBLAS workspace are
// accepted for source compatibility and ignored.
#ifndef PPLB200_PPL_KERNEL_LLM_CUDA_CUBLAS_GEMM_H
#define PPLB200_PPL_KERNEL_LLM_CUDA_CUBLAS_GEMM_H

#include "ppl/kernel/llm/cuda/common/general_include.h"
#include "ppl/kernel/llm/cuda/cublas/gemm_algo.h"
#include "ppl/common/types.h"
#include "ppl/common/log.h"
#include "pplb200_i8i8.h"

#include <cublasLt.h>

namespace ppl { namespace kernel { namespace llm { namespace cuda { namespace cublas {

// C[M,N] (int32, ldc) = A[M,K] (int8, row-major, lda) x B[N,K]^T (int8, row-major, ldb).
// Same argument checks and return codes as the reference (src/.../cublas/gemm.cu:196-215):
// transa must be false, transb true, types int8/int8/int32.  alpha must be 1 and beta 0 (the
// only values the linear ops pass, pmx/i8i8/column_parallel_linear.cu:111-112); `bias` (int32)
// must be null (idem, :108).
inline ppl::common::RetCode gemm_i8i8i32(
    const cudaStream_t stream,
    const cublasLtHandle_t& cublaslt_handle,
    const cublasLtMatmulAlgo_t* algo,
    const bool transa,
    const int64_t lda,
    const ppl::common::datatype_t typea,
    const void* A,
    const bool transb,
    const int64_t ldb,
    const ppl::common::datatype_t typeb,
    const void* B,
    const void* bias,
    const int64_t M,
    const int64_t N,
    const int64_t K,
    const int32_t alpha,
    const int32_t beta,
    const int64_t workspace_size,
    void* workspace,
    AlgoCache* algo_cache,
    const int64_t ldc,
    const ppl::common::datatype_t typec,
    void* C)
{
    (void)cublaslt_handle; (void)algo; (void)workspace_size; (void)workspace; (void)algo_cache;
    if (transa || !transb) {
        LOG(ERROR) << "only support transa = false and transb = true";
        return ppl::common::RC_UNSUPPORTED;
    }
    if (typea != ppl::common::DATATYPE_INT8 || typeb != ppl::common::DATATYPE_INT8 ||
        typec != ppl::common::DATATYPE_INT32) {
        LOG(ERROR) << "only support int8 x int8 -> int32";
        return ppl::common::RC_UNSUPPORTED;
    }
    if (alpha != 1 || beta != 0 || bias != nullptr) {
        LOG(ERROR) << "only support alpha = 1, beta = 0, no int32 bias";
        return ppl::common::RC_UNSUPPORTED;
    }
    return (ppl::common::RetCode)pplb200_i8i8_gemm(
        (pplb200_stream_t)stream, A, lda, B, ldb, M, N, K, PPLB200_EPI_RAW_I32, nullptr, nullptr, nullptr,
        0.0f, 0.0f, 0.0f, nullptr, 0, C, ldc, nullptr, nullptr);
}

// The COL32 / COL32_2R_4R4 / COL4_4R2_8C operand orders exist for the Turing / Ampere IMMA
// kernels of cuBLASLt (src/.../cublas/gemm.cu:365-488); there is no such path on sm_100a.
inline ppl::common::RetCode gemm_i8i8i32_col32(
    const cudaStream_t, const cublasLtHandle_t&, const void*, const void*,
    const int64_t, const int64_t, const int64_t, const bool, void*)
{
    LOG(ERROR) << "COL32 int8 GEMM is not available on sm_100a; use row-major operands";
    return ppl::common::RC_UNSUPPORTED;
}

}}}}}

#endif
