// The reference's cuBLASLt algorithm-cache types and the declaration of its algorithm search
// (include/ppl/kernel/llm/cuda/cublas/gemm_algo.h:31-141), kept so that every translation unit of a
// caller that includes cublas/gemm.h or cublas/gemm_algo.h -- the fp16 / fp8 linears as well --
// keeps compiling when this include directory shadows the reference's: same struct names and
// members, same key / hash / map types, same helper and function signatures.
//
// The sm_100a int8 GEMM is hand-written and has no algorithm search: the i8i8 operators accept an
// AlgoCache* and never touch it.  find_best_algo is declared only; its definition stays in the
// reference's own library (src/ppl/kernel/llm/cuda/cublas/gemm_algo.cu), which a caller that uses the
// fp16 / fp8 GEMMs links anyway.
#ifndef PPLB200_PPL_KERNEL_LLM_CUDA_CUBLAS_GEMM_ALGO_H
#define PPLB200_PPL_KERNEL_LLM_CUDA_CUBLAS_GEMM_ALGO_H

#include "ppl/kernel/llm/cuda/common/general_include.h"
#include "ppl/common/types.h"

#include <cublasLt.h>
#include <array>
#include <functional>
#include <unordered_map>
#include <utility>
#include <vector>

namespace ppl { namespace kernel { namespace llm { namespace cuda { namespace cublas {

struct MatmulDesc {
    cublasOperation_t transa;
    cublasOperation_t transb;
    bool operator==(const MatmulDesc& o) const { return transa == o.transa && transb == o.transb; }
};

struct MatrixLayout {
    cudaDataType_t datatype;
    cublasLtOrder_t layout;
    uint64_t rows;
    uint64_t cols;
    bool operator==(const MatrixLayout& o) const {
        return datatype == o.datatype && layout == o.layout && rows == o.rows && cols == o.cols;
    }
};

// key of the cache: the operation and its four matrix descriptors (A, B, C, D)
struct AlgoCacheIndex {
    MatmulDesc matmul_desc;
    std::array<MatrixLayout, 4> matrix_descs;
    bool operator==(const AlgoCacheIndex& o) const {
        return matmul_desc == o.matmul_desc && matrix_descs == o.matrix_descs;
    }
};

// Same mixing as the reference (field hashes shifted by their position and XOR-ed), written as a loop.
struct AlgoCacheIndexHash {
    std::size_t operator()(const AlgoCacheIndex& k) const {
        std::size_t h = std::hash<int>()(k.matmul_desc.transa) ^ (std::hash<int>()(k.matmul_desc.transb) << 1);
        int shift = 2;
        for (const MatrixLayout& m : k.matrix_descs) {
            h ^= std::hash<int>()(m.datatype) << shift++;
            h ^= std::hash<int>()(m.layout) << shift++;
            h ^= std::hash<uint64_t>()(m.rows) << shift++;
            h ^= std::hash<uint64_t>()(m.cols) << shift++;
        }
        return h;
    }
};

using AlgoCache = std::unordered_map<AlgoCacheIndex, cublasLtMatmulAlgo_t, AlgoCacheIndexHash>;

static inline MatmulDesc convert_matmul_desc(cublasLtMatmulDesc_t desc) {
    MatmulDesc m;
    size_t got = 0;
    cublasLtMatmulDescGetAttribute(desc, CUBLASLT_MATMUL_DESC_TRANSA, &m.transa, sizeof(m.transa), &got);
    cublasLtMatmulDescGetAttribute(desc, CUBLASLT_MATMUL_DESC_TRANSB, &m.transb, sizeof(m.transb), &got);
    return m;
}

static inline MatrixLayout convert_matrix_layout(cublasLtMatrixLayout_t desc) {
    MatrixLayout m;
    size_t got = 0;
    cublasLtMatrixLayoutGetAttribute(desc, CUBLASLT_MATRIX_LAYOUT_TYPE, &m.datatype, sizeof(m.datatype), &got);
    cublasLtMatrixLayoutGetAttribute(desc, CUBLASLT_MATRIX_LAYOUT_ORDER, &m.layout, sizeof(m.layout), &got);
    cublasLtMatrixLayoutGetAttribute(desc, CUBLASLT_MATRIX_LAYOUT_ROWS, &m.rows, sizeof(m.rows), &got);
    cublasLtMatrixLayoutGetAttribute(desc, CUBLASLT_MATRIX_LAYOUT_COLS, &m.cols, sizeof(m.cols), &got);
    return m;
}

// Defined by the reference's library (not by this one); not used on the i8i8 path.
std::pair<ppl::common::RetCode, cublasLtMatmulAlgo_t> find_best_algo(
    const cudaStream_t stream,
    const cublasLtHandle_t& lightHandle,
    const std::vector<int>& banned_algo_ids,
    cublasLtMatmulDesc_t computeDesc,
    const void* alpha,
    const void* A,
    cublasLtMatrixLayout_t Adesc,
    const void* B,
    cublasLtMatrixLayout_t Bdesc,
    const void* beta,
    const void* C,
    cublasLtMatrixLayout_t Cdesc,
    void* D,
    cublasLtMatrixLayout_t Ddesc,
    const int64_t workspace_size,
    void* workspace);

}}}}}

#endif
