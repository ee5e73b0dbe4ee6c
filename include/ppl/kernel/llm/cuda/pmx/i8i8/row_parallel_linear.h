// Row-parallel W8A8 linear with the reference's signature
// (include/ppl/kernel/llm/cuda/pmx/i8i8/row_parallel_linear.h:33-58), forwarded to the
// sm_100a implementation through the C ABI.
#ifndef PPLB200_PPL_KERNEL_LLM_CUDA_PMX_I8I8_ROW_PARALLEL_LINEAR_H
#define PPLB200_PPL_KERNEL_LLM_CUDA_PMX_I8I8_ROW_PARALLEL_LINEAR_H

#include "ppl/kernel/llm/cuda/common/general_include.h"
#include "ppl/kernel/llm/cuda/cublas/gemm.h"
#include "ppl/common/cuda/nccl_utils.h"
#include "ppl/common/log.h"

#include "quantize.h"

namespace ppl { namespace kernel { namespace llm { namespace cuda { namespace pmx { namespace i8i8 {

// How partial results of the K shards are combined when nccl_param->size > 1.
//   ROW_PARALLEL_REDUCE_INT32 (default): sum the int32 accumulators across ranks, then run the
//     dequant + bias epilogue once -- bit-identical to the unsharded linear.  Needs quant_buffer
//     (int32 [M, N]); every rank passes the same full-row scale_M and the same bias.
//   ROW_PARALLEL_REDUCE_FP16_REFERENCE: the reference's order -- dequantize each partial to fp16
//     (bias on rank 0 only) and all-reduce in fp16 (src/.../pmx/i8i8/row_parallel_linear.cu:84,131-158).
enum row_parallel_reduce_t {
    ROW_PARALLEL_REDUCE_INT32 = 0,
    ROW_PARALLEL_REDUCE_FP16_REFERENCE = 1,
};

// input int8 [.., K/size]; weight int8 [N, K/size] row-major; output fp16 [M, N] on every rank.
inline ppl::common::RetCode row_parallel_linear(
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
    const bool input_is_parallel,
    void* split_buffer,
    void* quant_buffer,
    const int64_t cublas_workspace_size,
    void* cublas_workspace,
    ppl::kernel::llm::cuda::cublas::AlgoCache* cublas_algo_cache,
    const ppl::common::TensorShape* output_shape,
    void* output,
    const row_parallel_reduce_t reduce = ROW_PARALLEL_REDUCE_INT32)
{
    (void)cublaslt_handle; (void)algo; (void)weight_shape; (void)split_buffer; (void)cublas_algo_cache; (void)output_shape;
    if (bias && bias_shape->GetDataType() != ppl::common::DATATYPE_FLOAT16) {
        LOG(ERROR) << "only support fp16 bias";
        return ppl::common::RC_UNSUPPORTED;
    }
    const int64_t M = (int64_t)input_shape->CalcElementsToDimensionExcludingPadding(input_shape->GetDimCount() - 1);
    return (ppl::common::RetCode)pplb200_i8i8_row_parallel_linear(
        (pplb200_stream_t)stream, input, M, /*input_ld=*/0, weight, bias, scale_M, scale_N, down_scale_M, down_scale_N,
        in_features, out_features, (int32_t)weight_layout, nccl_param->rank, nccl_param->size,
        (void*)nccl_param->comm, input_is_parallel ? 1 : 0, (int32_t)reduce, quant_buffer,
        cublas_workspace, cublas_workspace_size, output);
}

}}}}}}

#endif
