// Source-compatibility shim for the reference's cuBLASLt algorithm cache
// (include/ppl/kernel/llm/cuda/cublas/gemm_algo.h:31-91).  The sm_100a GEMM is hand-written and
// has no algorithm search, so the cache is accepted by the operators and never touched; it stays
// a default-constructible map type so that callers that own one keep compiling.
#ifndef PPLB200_PPL_KERNEL_LLM_CUDA_CUBLAS_GEMM_ALGO_H
#define PPLB200_PPL_KERNEL_LLM_CUDA_CUBLAS_GEMM_ALGO_H

#include "ppl/kernel/llm/cuda/common/general_include.h"
#include "ppl/common/types.h"

#include <cublasLt.h>
#include <unordered_map>

namespace ppl { namespace kernel { namespace llm { namespace cuda { namespace cublas {

// key: (M, N, K) bucket hash; value: unused here
using AlgoCache = std::unordered_map<uint64_t, cublasLtMatmulAlgo_t>;

}}}}}

#endif
