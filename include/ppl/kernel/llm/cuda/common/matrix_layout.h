// Matrix storage orders understood by the i8i8 operators.  The enumerator values are ABI
// (they cross the C boundary as int32) and equal the reference's
// (include/ppl/kernel/llm/cuda/common/matrix_layout.h:25-31); MatrixLayoutHelper keeps the
// reference's Init / GetOffset interface (:34-142) on top of one shared index function.
#ifndef PPLB200_PPL_KERNEL_LLM_CUDA_COMMON_MATRIX_LAYOUT_H
#define PPLB200_PPL_KERNEL_LLM_CUDA_COMMON_MATRIX_LAYOUT_H

#include "ppl/kernel/llm/cuda/common/general_include.h"

#if defined(__CUDACC__)
#define PPLB200_HD __host__ __device__
#else
#define PPLB200_HD
#endif

namespace ppl { namespace kernel { namespace llm { namespace cuda {

enum matrix_layout_t {
    MATRIX_LAYOUT_ROW_MAJOR = 0,
    MATRIX_LAYOUT_COL_MAJOR = 1,
    MATRIX_LAYOUT_COL32 = 2,        // cublasLt ORDER_COL32: panels of 32 columns, row-major inside a panel
    MATRIX_LAYOUT_COL32_2R_4R4 = 3, // cublasLt ORDER_COL32_2R_4R4 (Ampere IMMA weight order)
    MATRIX_LAYOUT_COL4_4R2_8C = 4,  // cublasLt ORDER_COL4_4R2_8C (Turing IMMA weight order)
};

// Element offset of (row, col) in a rows x cols matrix stored in `layout`.
PPLB200_HD inline int64_t MatrixLayoutOffset(matrix_layout_t layout, int64_t rows, int64_t cols, int64_t row, int64_t col) {
    const int64_t panel = (col >> 5) * rows * 32; // start of the 32-column panel (COL32 family)
    const int64_t c32 = col & 31;
    switch (layout) {
    case MATRIX_LAYOUT_ROW_MAJOR: return row * cols + col;
    case MATRIX_LAYOUT_COL_MAJOR: return col * rows + row;
    case MATRIX_LAYOUT_COL32: return panel + row * 32 + c32;
    case MATRIX_LAYOUT_COL32_2R_4R4: {
        const int64_t r32 = row & 31; // rows interleave inside blocks of 32: (r%8)/2, r/8, r%2
        const int64_t slot = ((((r32 & 7) >> 1) << 2) + (r32 >> 3)) * 2 + (r32 & 1);
        return panel + (row >> 5) * 1024 + slot * 32 + c32;
    }
    default: { // MATRIX_LAYOUT_COL4_4R2_8C: 8-row x 32-col blocks, split in 8x8, then 4x4 interleaved by row parity
        const int64_t line = (row & ~int64_t(7)) + ((row & 1) << 2) + (c32 >> 3);
        const int64_t quad = ((c32 & 4) ? 4 : 0) + ((row & 7) >> 1);
        return panel + line * 32 + quad * 4 + (c32 & 3);
    }
    }
}

template <matrix_layout_t layout>
struct MatrixLayoutHelper {
    int64_t rows = 0;
    int64_t cols = 0;

    PPLB200_HD inline void Init(const int64_t _rows, const int64_t _cols) {
        rows = _rows;
        cols = _cols;
    }
    PPLB200_HD inline int64_t GetOffset(const int64_t row_id, const int64_t col_id) const {
        return MatrixLayoutOffset(layout, rows, cols, row_id, col_id);
    }
};

}}}}

#endif
