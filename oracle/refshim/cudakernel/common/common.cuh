// TEST INFRASTRUCTURE ONLY.  Minimal stand-in for the one helper of
// ppl.kernel.cuda's cudakernel/common/common.cuh that the reference's i8i8
// sources use: a fixed-size vector copy.  It exists so the UNMODIFIED reference
// sources can be compiled into oracle/_ref as the parity comparator.
#ifndef PPLB200_REFSHIM_CUDAKERNEL_COMMON_CUH
#define PPLB200_REFSHIM_CUDAKERNEL_COMMON_CUH

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <vector>
#include <cub/cub.cuh>

template <int BYTES>
struct RefShimVec {};
template <> struct RefShimVec<2>  { typedef uint16_t type; };
template <> struct RefShimVec<4>  { typedef uint32_t type; };
template <> struct RefShimVec<8>  { typedef uint2 type; };
template <> struct RefShimVec<16> { typedef uint4 type; };

template <int BYTES>
__device__ __forceinline__ void copy(const void* src, void* dst) {
    typedef typename RefShimVec<BYTES>::type vec_t;
    *reinterpret_cast<vec_t*>(dst) = *reinterpret_cast<const vec_t*>(src);
}

#endif
