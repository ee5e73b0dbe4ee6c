// Common includes of the operator headers (same role as the reference's
// include/ppl/kernel/llm/cuda/common/general_include.h:18-27).
#ifndef PPLB200_PPL_KERNEL_LLM_CUDA_COMMON_GENERAL_INCLUDE_H
#define PPLB200_PPL_KERNEL_LLM_CUDA_COMMON_GENERAL_INCLUDE_H

#include "ppl/common/tensor_shape.h"
#include "ppl/common/retcode.h"

#include <stdint.h>
#include <cuda_runtime.h>

#endif
