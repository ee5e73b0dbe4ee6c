// Stand-in for ppl.common's types.h: the data-type tags and sizes used by the
// i8i8 linear path.  See retcode.h in this directory for why it exists.
#ifndef PPLB200_COMPAT_PPL_COMMON_TYPES_H
#define PPLB200_COMPAT_PPL_COMMON_TYPES_H

#include <stdint.h>

namespace ppl { namespace common {

typedef uint32_t datatype_t;

enum {
    DATATYPE_UNKNOWN = 0,
    DATATYPE_UINT8 = 1,
    DATATYPE_UINT16 = 2,
    DATATYPE_UINT32 = 3,
    DATATYPE_UINT64 = 4,
    DATATYPE_FLOAT16 = 5,
    DATATYPE_FLOAT32 = 6,
    DATATYPE_FLOAT64 = 7,
    DATATYPE_BFLOAT16 = 8,
    DATATYPE_INT4B = 9,
    DATATYPE_INT8 = 10,
    DATATYPE_INT16 = 11,
    DATATYPE_INT32 = 12,
    DATATYPE_INT64 = 13,
    DATATYPE_BOOL = 14,
    DATATYPE_COMPLEX64 = 15,
    DATATYPE_COMPLEX128 = 16,
    DATATYPE_FLOAT8E4M3 = 17,
    DATATYPE_FLOAT8E5M2 = 18,
    DATATYPE_MAX,
};

static inline uint32_t GetSizeOfDataType(datatype_t dt) {
    static const uint32_t sizes[] = {0, 1, 2, 4, 8, 2, 4, 8, 2, 1, 1, 2, 4, 8, 1, 8, 16, 1, 1};
    return dt < DATATYPE_MAX ? sizes[dt] : 0;
}

}}

#endif
