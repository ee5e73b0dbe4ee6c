// Stand-in for ppl.common's retcode.h, which is not part of the kernel library's
// tree (it is fetched at configure time by the reference's build).  Only the
// surface the i8i8 linear path touches.  In a real deployment put ppl.common's
// own include directory BEFORE this one on the include path; the numeric values
// below follow ppl.common's published enum order.
#ifndef PPLB200_COMPAT_PPL_COMMON_RETCODE_H
#define PPLB200_COMPAT_PPL_COMMON_RETCODE_H

#include <stdint.h>

namespace ppl { namespace common {

typedef uint32_t RetCode;

enum {
    RC_SUCCESS = 0,
    RC_OTHER_ERROR,
    RC_UNSUPPORTED,
    RC_OUT_OF_MEMORY,
    RC_INVALID_VALUE,
    RC_EXISTS,
    RC_NOT_FOUND,
    RC_PERMISSION_DENIED,
    RC_HOST_MEMORY_ERROR,
    RC_DEVICE_MEMORY_ERROR,
    RC_DEVICE_RUNTIME_ERROR,
    RC_OUT_OF_RANGE,
};

static inline const char* GetRetCodeStr(RetCode rc) {
    static const char* names[] = {
        "success", "other error", "unsupported", "out of memory", "invalid value", "already exists",
        "not found", "permission denied", "host memory error", "device memory error",
        "device runtime error", "out of range",
    };
    return rc < sizeof(names) / sizeof(names[0]) ? names[rc] : "unknown";
}

}}

#endif
