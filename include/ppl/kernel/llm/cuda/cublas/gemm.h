// GEMM entry points with the reference's signatures (include/ppl/kernel/llm/cuda/cublas/gemm.h:32-124).
//
//  * gemm_i8i8i32 / gemm_i8i8i32_col32 -- the int8 path -- are provided here, forwarded to the sm_100a
//    tcgen05 kernel through the C ABI.  They have internal linkage (static inline), so a program that also
//    links the reference's library keeps calling these from every translation unit that includes this header;
//    the two never clash at link time.  cuBLASLt handle, algorithm, algorithm cache and cuBLAS workspace are
//    accepted for source compatibility and ignored.
//  * gemm (fp16 / bf16) and gemm_fp8 are declared exactly as the reference declares them and stay defined by
//    the reference's own library (src/ppl/kernel/llm/cuda/cublas/gemm.cu:31-169, :490-...): this library does
//    not replace them, and the fp16 / fp8 linears of a caller keep compiling and linking as before.
#ifndef PPLB200_PPL_KERNEL_LLM_CUDA_CUBLAS_GEMM_H
#define PPLB200_PPL_KERNEL_LLM_CUDA_CUBLAS_GEMM_H

#include "ppl/kernel/llm/cuda/common/general_include.h"
#include "ppl/kernel/llm/cuda/cublas/gemm_algo.h"
#include "ppl/common/types.h"
#include "ppl/common/log.h"
#include "pplb200_i8i8.h"

#include <cublasLt.h>

namespace ppl { namespace kernel { namespace llm { namespace cuda { namespace cublas {

// Row-major GEMM over cuBLASLt for fp16 / bf16 operands: the reference's, not replaced.
ppl::common::RetCode gemm(
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
    const float alpha,
    const float beta,
    const int64_t workspace_size,
    void* workspace,
    const int64_t ldc,
    const ppl::common::datatype_t typec,
    void* C);

// C[M,N] (int32, ldc) = alpha * (A[M,K] (int8, row-major, lda) x B[N,K]^T (int8, row-major, ldb)) + beta * C
// (+ bias[n], int32, when bias != nullptr), all in wrapping int32 arithmetic as cuBLASLt's CUBLAS_COMPUTE_32I
// with an int32 scale type computes it (src/.../cublas/gemm.cu:187-188,239-243,329-345).
// Same argument checks and return codes as the reference (:196-215): transa must be false, transb true,
// types int8 / int8 / int32.
static inline ppl::common::RetCode gemm_i8i8i32(
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
    if (typea != ppl::common::DATATYPE_INT8) {
        LOG(ERROR) << "only support int8 A matrix";
        return ppl::common::RC_UNSUPPORTED;
    }
    if (typeb != ppl::common::DATATYPE_INT8) {
        LOG(ERROR) << "only support int8 B matrix";
        return ppl::common::RC_UNSUPPORTED;
    }
    if (typec != ppl::common::DATATYPE_INT32) {
        LOG(ERROR) << "only support int32 C matrix";
        return ppl::common::RC_UNSUPPORTED;
    }
    if (transa != false) {
        LOG(ERROR) << "only support non-transposed A matrix";
        return ppl::common::RC_UNSUPPORTED;
    }
    if (transb != true) {
        LOG(ERROR) << "only support transposed B matrix";
        return ppl::common::RC_UNSUPPORTED;
    }
    return (ppl::common::RetCode)pplb200_i8i8_gemm_i32(
        (pplb200_stream_t)stream, A, lda, B, ldb, M, N, K, alpha, beta, bias, C, ldc);
}

// The COL32 / COL32_2R_4R4 / COL4_4R2_8C operand orders exist for the Turing / Ampere IMMA
// kernels of cuBLASLt (src/.../cublas/gemm.cu:365-488); the tensor cores of sm_100a have no such path.
// Operands in those orders are served by the linear operators, which re-lay them out (see
// pplb200_i8i8_relayout); this raw entry point stays unsupported.
static inline ppl::common::RetCode gemm_i8i8i32_col32(
    const cudaStream_t, const cublasLtHandle_t&, const void*, const void*,
    const int64_t, const int64_t, const int64_t, const bool, void*)
{
    LOG(ERROR) << "COL32 int8 GEMM is not available on sm_100a; use row-major operands";
    return ppl::common::RC_UNSUPPORTED;
}

#ifdef PPLNN_ENABLE_FP8
// fp8 x fp8 -> fp16 over cuBLASLt: the reference's, not replaced.
ppl::common::RetCode gemm_fp8(
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
    const float alpha,
    const float beta,
    const int64_t workspace_size,
    void* workspace,
    const int64_t ldc,
    const ppl::common::datatype_t typec,
    void* C);
#endif

}}}}}

#endif
