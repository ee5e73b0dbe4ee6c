// Device helpers shared by the per-token quantizers: streaming 128-bit loads, the block-wide
// maximum, and the 16-element rounding step (bit-identical to rn(v / scale) with IEEE division).
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace pplb200 {
namespace qdev {

constexpr int QTPB = 256;

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ float block_max(float v, float* red, int nwarps) {
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
    for (int w = 1; w < nwarps; ++w) r = fmaxf(r, red[w]);
    return r;
}

// Quantizes 16 consecutive halves to 16 int8 (one 128-bit store): q = rn(v / scale), identical to
// __float2int_rn(__fdiv_rn(v, scale)).  v * (1/scale) is within a few ulp of the IEEE quotient, so both
// round to the same integer unless the product sits next to a half-integer.  The common path uses
// only full-rate arithmetic: adding 1.5 * 2^23 rounds the product to the nearest-even integer and
// leaves that integer's two's-complement byte in the low mantissa bits; subtracting it back gives
// the rounding residual, and the group is redone with exact divisions only if some residual is
// within 2^-12 of one half (or is not a number: NaN / infinite inputs take the exact path too).
__device__ __forceinline__ uint4 quant16(const __half2* h, float scale, float inv_scale) {
    constexpr float kMagic = 12582912.0f; // 1.5 * 2^23
    float f[16];
    uint32_t b[16];
    bool safe = true;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float2 v = __half22float2(h[i]);
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float t = f[i] * inv_scale;
        const float u = __fadd_rn(t, kMagic);
        const float resid = __fsub_rn(t, __fsub_rn(u, kMagic));
        b[i] = __float_as_uint(u);
        safe = safe && (fabsf(resid) < 0.5f - 1.0f / 4096.0f);
    }
    if (!safe) {
#pragma unroll
        for (int i = 0; i < 16; ++i) b[i] = (uint32_t)__float2int_rn(__fdiv_rn(f[i], scale));
    }
    uint4 o;
    o.x = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
    o.y = __byte_perm(__byte_perm(b[4], b[5], 0x0040), __byte_perm(b[6], b[7], 0x0040), 0x5410);
    o.z = __byte_perm(__byte_perm(b[8], b[9], 0x0040), __byte_perm(b[10], b[11], 0x0040), 0x5410);
    o.w = __byte_perm(__byte_perm(b[12], b[13], 0x0040), __byte_perm(b[14], b[15], 0x0040), 0x5410);
    return o;
}

} // namespace qdev
} // namespace pplb200
