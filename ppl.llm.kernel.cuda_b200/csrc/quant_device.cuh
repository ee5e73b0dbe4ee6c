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

// Block-wide maximum plus a block-wide OR of `flag` (one barrier for both).
__device__ __forceinline__ float block_max_any(float v, bool flag, float* red, int nwarps, bool& any) {
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[warp] = v;
    any = __syncthreads_or(flag ? 1 : 0) != 0;
    float r = red[0];
    for (int w = 1; w < nwarps; ++w) r = fmaxf(r, red[w]);
    return r;
}

// max |x| over `n2` packed halves.  The fold propagates NaNs (same cost as dropping them), so a NaN anywhere is
// seen in the result; only then is the fold redone dropping NaNs, as the reference's fmax chain does
// (src/ppl/kernel/llm/cuda/pmx/i8i8/quantize.cu:47-57).  Returns the NaN-free maximum; `saw_nan` says whether a NaN occurred.
__device__ __forceinline__ float absmax_halves(const __half2* h, int n2, bool& saw_nan) {
    __half2 m2 = __float2half2_rn(0.0f);
    for (int i = 0; i < n2; ++i) m2 = __hmax2_nan(m2, __habs2(h[i]));
    saw_nan = __hisnan(__low2half(m2)) || __hisnan(__high2half(m2));
    if (saw_nan) {
        m2 = __float2half2_rn(0.0f);
        for (int i = 0; i < n2; ++i) m2 = __hmax2(m2, __habs2(h[i]));
    }
    return fmaxf(__low2float(m2), __high2float(m2));
}

// Per-row constants of the rounding step.
struct QuantRow {
    float scale;   // max(amax / 127, 1e-7), what the reference divides by
    float inv_hi;  // (1 / scale) nudged up and down by 2^-21: v * inv_lo <= v / scale <= v * inv_hi for v >= 0
    float inv_lo;
    bool exact;    // row holds a NaN or its maximum is infinite: every element takes the IEEE division
};
__device__ __forceinline__ QuantRow make_quant_row(float amax, bool saw_nan) {
    QuantRow q;
    q.scale = fmaxf(__fdiv_rn(amax, 127.0f), 1e-7f);
    const float inv = __frcp_rn(q.scale);
    q.inv_hi = __fmul_rn(inv, 1.0f + 0x1p-21f);
    q.inv_lo = __fmul_rn(inv, 1.0f - 0x1p-21f);
    q.exact = saw_nan || !(amax < __int_as_float(0x7f800000));
    return q;
}

// Quantizes 16 consecutive halves to 16 int8 (one 128-bit store): q = rn(v / scale), identical to
// __float2int_rn(__fdiv_rn(v, scale)) (quantize.cu:72).  Fast path, three full-rate instructions per element:
// fma(v, inv_hi, M) and fma(v, inv_lo, M) with M = 1.5 * 2^23 round the two products -- which bracket the IEEE
// quotient, rounding errors of the reciprocal and of the division included (both below 2^-23 relative, the
// bracket is 2^-22 wide on each side) -- to the nearest-even integer and leave that integer's two's-complement
// byte in the low mantissa bits.  Rounding to an integer is monotone, so when both results agree every value in
// the bracket, the quotient among them, rounds to that integer.  When they differ for some element of the group
// (the quotient lies within ~1e-4 of a half-integer: about one group in a thousand), or when the row is flagged
// `exact`, the group is redone with IEEE divisions.  CHECK_NAN: the caller did not scan the row itself (row
// maximum given), so NaN elements, whose two fma results would agree, are looked for here.
template <bool CHECK_NAN>
__device__ __forceinline__ uint4 quant16(const __half2* h, const QuantRow& row) {
    constexpr float kMagic = 12582912.0f; // 1.5 * 2^23
    float f[16];
    uint32_t b[16];
    uint32_t differ = row.exact ? 1u : 0u;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float2 v = __half22float2(h[i]);
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
        if (CHECK_NAN && (__hisnan(__low2half(h[i])) || __hisnan(__high2half(h[i])))) differ = 1u;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        b[i] = __float_as_uint(__fmaf_rn(f[i], row.inv_hi, kMagic));
        differ |= b[i] ^ __float_as_uint(__fmaf_rn(f[i], row.inv_lo, kMagic));
    }
    if (differ != 0u) {
#pragma unroll
        for (int i = 0; i < 16; ++i) b[i] = (uint32_t)__float2int_rn(__fdiv_rn(f[i], row.scale));
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
