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
//   ROW_PARALLEL_REDUCE_FP16_REFERENCE (default of the overload with the reference's argument list): the
//     reference's order -- dequantize each partial to fp16 with THIS rank's scale_M (bias on rank 0 only) and
//     all-reduce in fp16 (src/.../pmx/i8i8/row_parallel_linear.cu:84,131-158).  This is what an unchanged
//     caller expects: it quantizes each K shard on its own rank, so scale_M differs from rank to rank.
//   ROW_PARALLEL_REDUCE_INT32 (opt-in): sum the int32 accumulators across ranks, then run the dequant + bias
//     epilogue once -- bit-identical to the unsharded linear.  Only meaningful when every rank passes the SAME
//     full-row scale_M (activations quantized with the maximum over the whole row, e.g. by
//     minmax_quantize_fp16_sharded below) and the same bias; needs quant_buffer (int32 [M, N]).
enum row_parallel_reduce_t {
    ROW_PARALLEL_REDUCE_INT32 = 0,
    ROW_PARALLEL_REDUCE_FP16_REFERENCE = 1,
};

// input int8 [.., K/size]; weight int8 [N, K/size] row-major; output fp16 [M, N] on every rank.
static inline ppl::common::RetCode row_parallel_linear(
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
    const row_parallel_reduce_t reduce = ROW_PARALLEL_REDUCE_FP16_REFERENCE)
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

// The same operator with the reduction over peer-mapped memory instead of a collective library
// (ranks of one NVLink domain): `p2p_context` is a context of pplb200_p2p_create that has been
// connected to its peers; it replaces nccl_param, quant_buffer and the cuBLAS arguments.  Result
// and argument meaning as ROW_PARALLEL_REDUCE_INT32; M must be divisible by the number of ranks
// (RC_UNSUPPORTED otherwise: call the overload above).  No counterpart in the reference.
static inline ppl::common::RetCode row_parallel_linear(
    const cudaStream_t stream,
    void* p2p_context,
    const ppl::common::TensorShape* input_shape,
    const void* input,
    const ppl::common::TensorShape* bias_shape,
    const void* bias,
    const void* scale_M,
    const void* scale_N,
    const float down_scale_M,
    const float down_scale_N,
    const int64_t in_features,
    const int64_t out_features,
    const void* weight,
    void* output)
{
    if (bias && bias_shape->GetDataType() != ppl::common::DATATYPE_FLOAT16) {
        LOG(ERROR) << "only support fp16 bias";
        return ppl::common::RC_UNSUPPORTED;
    }
    const int64_t M = (int64_t)input_shape->CalcElementsToDimensionExcludingPadding(input_shape->GetDimCount() - 1);
    return (ppl::common::RetCode)pplb200_i8i8_row_parallel_linear_p2p(
        (pplb200_stream_t)stream, p2p_context, input, M, /*input_ld=*/0, weight, bias, scale_M, scale_N, down_scale_M,
        down_scale_N, in_features, out_features, /*phases=*/7, output);
}

// Per-token quantizer for activations sharded along the quantized dimension (what the preceding
// column-parallel operator leaves on each rank): int8 values and full-row scales equal those of
// minmax_quantize_fp16 on the unsharded rows.  input_shape is the shard's shape [.., K / size].
static inline ppl::common::RetCode minmax_quantize_fp16_sharded(
    const cudaStream_t stream,
    void* p2p_context,
    const ppl::common::TensorShape* input_shape,
    const void* input,
    const float up_scale,
    void* quantized,
    void* scale)
{
    const int64_t dim = input_shape->GetDim(input_shape->GetDimCount() - 1);
    const int64_t batch = (int64_t)input_shape->CalcElementsToDimensionExcludingPadding(input_shape->GetDimCount() - 1);
    return (ppl::common::RetCode)pplb200_i8i8_minmax_quantize_fp16_p2p((pplb200_stream_t)stream, p2p_context, input, batch,
                                                                       dim, up_scale, /*phases=*/3, quantized, scale);
}

}}}}}}

#endif
