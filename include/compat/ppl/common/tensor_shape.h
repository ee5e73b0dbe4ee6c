// Stand-in for ppl.common's TensorShape: dims + data type, and the element-count
// helper the linear ops use to derive M.  See retcode.h in this directory.
#ifndef PPLB200_COMPAT_PPL_COMMON_TENSOR_SHAPE_H
#define PPLB200_COMPAT_PPL_COMMON_TENSOR_SHAPE_H

#include "ppl/common/types.h"

#include <initializer_list>
#include <vector>

namespace ppl { namespace common {

class TensorShape final {
public:
    TensorShape() {}
    TensorShape(datatype_t dt, std::initializer_list<int64_t> dims) : data_type_(dt), dims_(dims) {}

    void SetDataType(datatype_t dt) { data_type_ = dt; }
    datatype_t GetDataType() const { return data_type_; }

    void Reshape(std::initializer_list<int64_t> dims) { dims_.assign(dims.begin(), dims.end()); }
    void Reshape(const int64_t* dims, uint32_t n) { dims_.assign(dims, dims + n); }
    uint32_t GetDimCount() const { return (uint32_t)dims_.size(); }
    int64_t GetDim(uint32_t i) const { return dims_[i]; }

    // product of dims [0, end)
    uint64_t CalcElementsToDimensionExcludingPadding(uint32_t end) const {
        uint64_t n = 1;
        for (uint32_t i = 0; i < end && i < dims_.size(); ++i) n *= (uint64_t)dims_[i];
        return n;
    }
    uint64_t CalcElementsExcludingPadding() const {
        return CalcElementsToDimensionExcludingPadding((uint32_t)dims_.size());
    }

private:
    datatype_t data_type_ = DATATYPE_UNKNOWN;
    std::vector<int64_t> dims_;
};

}}

#endif
