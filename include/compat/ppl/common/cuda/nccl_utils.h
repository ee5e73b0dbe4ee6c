// Stand-in for ppl.common's cuda/nccl_utils.h: the communicator handle the
// tensor-parallel linears receive, and the two collectives they call.
// See ../retcode.h in this directory tree.
#ifndef PPLB200_COMPAT_PPL_COMMON_CUDA_NCCL_UTILS_H
#define PPLB200_COMPAT_PPL_COMMON_CUDA_NCCL_UTILS_H

#include "ppl/common/retcode.h"
#include "ppl/common/log.h"

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <nccl.h>
#include <type_traits>

namespace ppl { namespace common {

struct NcclParam {
    int rank = 0;
    int size = 1;
    ncclComm_t comm = nullptr;
};

template <typename T>
inline ncclDataType_t GetNcclDataType() {
    if (std::is_same<T, half>::value) return ncclHalf;
    if (std::is_same<T, float>::value) return ncclFloat;
    if (std::is_same<T, int32_t>::value) return ncclInt32;
    if (std::is_same<T, int8_t>::value) return ncclInt8;
    return ncclUint8;
}

template <typename T>
inline RetCode NcclAllReduceSum(const T* send, T* recv, size_t count, const NcclParam* p, cudaStream_t stream) {
    if (p->size == 1) return RC_SUCCESS;
    ncclResult_t r = ncclAllReduce(send, recv, count, GetNcclDataType<T>(), ncclSum, p->comm, stream);
    if (r != ncclSuccess) {
        LOG(ERROR) << "ncclAllReduce failed: " << ncclGetErrorString(r);
        return RC_DEVICE_RUNTIME_ERROR;
    }
    return RC_SUCCESS;
}

template <typename T>
inline RetCode NcclAllGather(const T* send, T* recv, size_t count, const NcclParam* p, cudaStream_t stream) {
    if (p->size == 1) return RC_SUCCESS;
    ncclResult_t r = ncclAllGather(send, recv, count, GetNcclDataType<T>(), p->comm, stream);
    if (r != ncclSuccess) {
        LOG(ERROR) << "ncclAllGather failed: " << ncclGetErrorString(r);
        return RC_DEVICE_RUNTIME_ERROR;
    }
    return RC_SUCCESS;
}

}}

#endif
