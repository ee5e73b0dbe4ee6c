// TEST INFRASTRUCTURE ONLY.  Declaration stand-in for ppl.kernel.cuda's batched
// [d0, d1, d2] -> [d1, d0, d2] transpose, which the reference's column-parallel
// linear calls after its all-gather.  Defined in ref_capi.cu.
#ifndef PPLB200_REFSHIM_CUDAKERNEL_TRANSPOSE_H
#define PPLB200_REFSHIM_CUDAKERNEL_TRANSPOSE_H

#include "ppl/common/retcode.h"
#include "ppl/common/types.h"
#include <cuda_runtime.h>
#include <stdint.h>

ppl::common::RetCode PPLCUDATranspose01ForwardImp(
    cudaStream_t stream, const void* input, ppl::common::datatype_t dtype,
    int64_t dim0, int64_t dim1, int64_t dim2, void* output);

#endif
