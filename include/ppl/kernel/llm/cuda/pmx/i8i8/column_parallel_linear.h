// Column-parallel W8A8 linear with the reference's signature
// (include/ppl/kernel/llm/cuda/pmx/i8i8/column_parallel_linear.h:33-58), forwarded to the
// sm_100a implementation through the C ABI.
#ifndef PPLB200_PPL_KERNEL_LLM_CUDA_PMX_I8I8_COLUMN_PARALLEL_LINEAR_H
#define PPLB200_PPL_KERNEL_LLM_CUDA_PMX_I8I8_COLUMN_PARALLEL_LINEAR_H

#include "ppl/kernel/llm/cuda/common/general_include.h"
#include "ppl/kernel/llm/cuda/cublas/gemm.h"
#include "ppl/common/cuda/nccl_utils.h"
#include "ppl/common/log.h"

#include "quantize.h"

namespace ppl { namespace kernel { namespace llm { namespace cuda { namespace pmx { namespace i8i8 {

// input int8 [.., K]; weight int8 [N/size, K] row-major; output:
//   gather_output == false -> RAW int32 [M, N/size] (no dequant), as the reference
//   gather_output == true  -> fp16 [M, N] (all-gathered over the communicator when size > 1)
// cublasLt handle / algo / algo cache / cuBLAS workspace are accepted and ignored; quant_buffer
// is not needed (the int32 accumulators stay in tensor memory) but accepted.
static inline ppl::common::RetCode column_parallel_linear(
    const cudaStream_t stream,
    const cublasLtHandle_t& cublaslt_handle,
    const cublasLtMatmulAlgo_t* algo,
    const ppl::common::TensorShape* input_shape,
    const void* input,
    const ppl::common::TensorShape* weight_shape,
    const void* weight,
    const ppl::common::TensorShape* bias_shape,
    const void* bias,
    const void* scale_M,
    const void* scale_N,
    const float down_scale_M,
    const float down_scale_N,
    const int64_t in_features,
    const int64_t out_features,
    const matrix_layout_t weight_layout,
    const ppl::common::NcclParam* nccl_param,
    const bool gather_output,
    void* gather_buffer,
    void* quant_buffer,
    const int64_t cublas_workspace_size,
    void* cublas_workspace,
    ppl::kernel::llm::cuda::cublas::AlgoCache* cublas_algo_cache,
    const ppl::common::TensorShape* output_shape,
    void* output)
{
    (void)cublaslt_handle; (void)algo; (void)weight_shape; (void)cublas_algo_cache; (void)output_shape;
    if (bias && bias_shape->GetDataType() != ppl::common::DATATYPE_FLOAT16) {
        LOG(ERROR) << "only support fp16 bias";
        return ppl::common::RC_UNSUPPORTED;
    }
    const int64_t M = (int64_t)input_shape->CalcElementsToDimensionExcludingPadding(input_shape->GetDimCount() - 1);
    return (ppl::common::RetCode)pplb200_i8i8_column_parallel_linear(
        (pplb200_stream_t)stream, input, M, weight, bias, scale_M, scale_N, down_scale_M, down_scale_N,
        in_features, out_features, (int32_t)weight_layout, nccl_param->rank, nccl_param->size,
        (void*)nccl_param->comm, gather_output ? 1 : 0, gather_buffer, quant_buffer,
        cublas_workspace, cublas_workspace_size, output);
}

// The same operator with gather_output = true done over peer-mapped memory instead of NcclAllGather + transpose:
// the GEMM epilogues of all ranks store their fp16 tiles straight into every rank's [M, N] matrix (see
// pplb200_i8i8_column_parallel_linear_p2p).  `p2p_context` is a connected context of pplb200_p2p_create; it
// replaces nccl_param, gather_buffer, quant_buffer and the cuBLAS arguments.  No counterpart in the reference.
static inline ppl::common::RetCode column_parallel_linear(
    const cudaStream_t stream,
    void* p2p_context,
    const ppl::common::TensorShape* input_shape,
    const void* input,
    const void* weight,
    const ppl::common::TensorShape* bias_shape,
    const void* bias,
    const void* scale_M,
    const void* scale_N,
    const float down_scale_M,
    const float down_scale_N,
    const int64_t in_features,
    const int64_t out_features,
    void* output)
{
    if (bias && bias_shape->GetDataType() != ppl::common::DATATYPE_FLOAT16) {
        LOG(ERROR) << "only support fp16 bias";
        return ppl::common::RC_UNSUPPORTED;
    }
    const int64_t M = (int64_t)input_shape->CalcElementsToDimensionExcludingPadding(input_shape->GetDimCount() - 1);
    return (ppl::common::RetCode)pplb200_i8i8_column_parallel_linear_p2p(
        (pplb200_stream_t)stream, p2p_context, input, M, weight, bias, scale_M, scale_N, down_scale_M, down_scale_N,
        in_features, out_features, /*phases=*/3, output);
}

}}}}}}

#endif
