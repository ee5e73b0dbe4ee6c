// Per-token quantize / dequantize operators with the reference's names, argument order and
// scale conventions (include/ppl/kernel/llm/cuda/pmx/i8i8/quantize.h:26-55), forwarded to the
// sm_100a kernels through the C ABI.
#ifndef PPLB200_PPL_KERNEL_LLM_CUDA_PMX_I8I8_QUANTIZE_H
#define PPLB200_PPL_KERNEL_LLM_CUDA_PMX_I8I8_QUANTIZE_H

#include "ppl/kernel/llm/cuda/common/general_include.h"
#include "ppl/kernel/llm/cuda/common/matrix_layout.h"
#include "pplb200_i8i8.h"

namespace ppl { namespace kernel { namespace llm { namespace cuda { namespace pmx { namespace i8i8 {

// fp16 scale vectors store scale * up_scale so that small scales stay clear of fp16 subnormals;
// the dequantizer multiplies by the matching down scale.
constexpr float token_up_scale = 4096.0f;
constexpr float hidden_up_scale = 8192.0f;
constexpr float token_down_scale = 1.0f / 4096.0f;
constexpr float hidden_down_scale = 1.0f / 8192.0f;

static inline ppl::common::RetCode minmax_quantize_fp16(
    cudaStream_t stream,
    const void* input,           // fp16, [batch, quant_dim]
    const int64_t batch,
    const int64_t quant_dim,
    const float up_scale,        // scale[i] = scale_val * up_scale
    const matrix_layout_t to_layout,
    void* quantized,             // int8, [batch, quant_dim]
    void* scale)                 // fp16, [batch]
{
    return (ppl::common::RetCode)pplb200_i8i8_minmax_quantize_fp16(
        (pplb200_stream_t)stream, input, batch, quant_dim, up_scale, (int32_t)to_layout, quantized, scale);
}

static inline ppl::common::RetCode minmax_dequantize_fp16(
    cudaStream_t stream,
    const void* input,              // int32, [batch, quant_dim] in from_layout
    const void* optional_bias,      // fp16, [quant_dim]
    const void* scale_per_batch,    // fp16, [batch]
    const void* scale_per_channel,  // fp16, [quant_dim]
    const int64_t batch,
    const int64_t quant_dim,
    const float down_scale_batch,
    const float down_scale_channel,
    const matrix_layout_t from_layout,
    void* output)                   // fp16, [batch, quant_dim]
{
    return (ppl::common::RetCode)pplb200_i8i8_minmax_dequantize_fp16(
        (pplb200_stream_t)stream, input, optional_bias, scale_per_batch, scale_per_channel, batch, quant_dim,
        down_scale_batch, down_scale_channel, (int32_t)from_layout, output);
}

// Consumers of the raw int32 GEMM output; reference declarations quantize.h:57-126.
static inline ppl::common::RetCode minmax_dequantize_split3_fp16(
    cudaStream_t stream, const void* input, const void* optional_bias, const void* scale_per_batch,
    const void* scale_per_channel, const int64_t batch, const int64_t quant_dim, const int64_t split_dim_0,
    const int64_t split_dim_1, const int64_t split_dim_2, const float down_scale_batch, const float down_scale_channel,
    const matrix_layout_t from_layout, void* output_0, void* output_1, void* output_2)
{
    return (ppl::common::RetCode)pplb200_i8i8_minmax_dequantize_split3_fp16(
        (pplb200_stream_t)stream, input, optional_bias, scale_per_batch, scale_per_channel, batch, quant_dim, split_dim_0,
        split_dim_1, split_dim_2, down_scale_batch, down_scale_channel, (int32_t)from_layout, output_0, output_1, output_2);
}

static inline ppl::common::RetCode minmax_dequantize_silu_fp16(
    cudaStream_t stream, const void* input, const void* input_scale_per_batch, const void* input_scale_per_channel,
    const void* optional_gate, const void* gate_scale_per_batch, const void* gate_scale_per_channel, const int64_t batch,
    const int64_t quant_dim, const matrix_layout_t from_layout, float down_scale_batch, float down_scale_channel,
    void* output)
{
    return (ppl::common::RetCode)pplb200_i8i8_minmax_dequantize_silu_fp16(
        (pplb200_stream_t)stream, input, input_scale_per_batch, input_scale_per_channel, optional_gate, gate_scale_per_batch,
        gate_scale_per_channel, batch, quant_dim, (int32_t)from_layout, down_scale_batch, down_scale_channel, output);
}

static inline ppl::common::RetCode minmax_requantize_silu_fp16(
    cudaStream_t stream, const void* input, const void* input_scale_per_batch, const void* input_scale_per_channel,
    const void* optional_gate, const void* gate_scale_per_batch, const void* gate_scale_per_channel, const int64_t batch,
    const int64_t quant_dim, const matrix_layout_t layout, const float up_scale, const float down_scale_batch,
    const float down_scale_channel, void* workspace, void* output, void* scale)
{
    return (ppl::common::RetCode)pplb200_i8i8_minmax_requantize_silu_fp16(
        (pplb200_stream_t)stream, input, input_scale_per_batch, input_scale_per_channel, optional_gate, gate_scale_per_batch,
        gate_scale_per_channel, batch, quant_dim, (int32_t)layout, up_scale, down_scale_batch, down_scale_channel, workspace,
        output, scale);
}

static inline ppl::common::RetCode minmax_requantize_swiglu_fp16(
    cudaStream_t stream, const void* input, const void* input_scale_per_batch, const void* input_scale_per_channel,
    const int64_t batch, const int64_t quant_dim, const float beta, const matrix_layout_t layout, const float up_scale,
    const float down_scale_batch, const float down_scale_channel, void* workspace, void* output, void* scale)
{
    return (ppl::common::RetCode)pplb200_i8i8_minmax_requantize_swiglu_fp16(
        (pplb200_stream_t)stream, input, input_scale_per_batch, input_scale_per_channel, batch, quant_dim, beta,
        (int32_t)layout, up_scale, down_scale_batch, down_scale_channel, workspace, output, scale);
}

// input + skip -> skip_out; quantize(rmsnorm(input + skip) * weight) -> output, output_scale
// (reference: include/ppl/kernel/llm/cuda/pmx/i8i8/quantize.h:128-141).
static inline ppl::common::RetCode skip_rmsnorm_minmax_quantize_fp16(
    const cudaStream_t stream,
    const void* input,            // [batch, hidden dim]
    const void* weight,           // [hidden dim]
    const void* skip,             // [batch, hidden dim] or null
    const float eps,
    const int64_t batch,
    const int64_t normalize_shape,
    const float up_scale,
    const matrix_layout_t to_layout,
    void* skip_out,               // [batch, hidden dim]
    void* output_scale,           // [batch]
    void* output)                 // [batch, hidden dim]
{
    return (ppl::common::RetCode)pplb200_i8i8_skip_rmsnorm_minmax_quantize_fp16(
        (pplb200_stream_t)stream, input, weight, skip, eps, batch, normalize_shape, up_scale, (int32_t)to_layout,
        skip_out, output_scale, output);
}

}}}}}}

#endif
