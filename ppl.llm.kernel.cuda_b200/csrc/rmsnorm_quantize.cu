// Fused skip-add + RMSNorm + per-token int8 quantize: the producer that feeds the W8A8 linear in
// a transformer block (it replaces the stand-alone activation quantizer there).
// Reference: src/ppl/kernel/llm/cuda/pmx/i8i8/rms_norm.cu:40-302 (kernels :40-182, launcher :186-302),
// declaration include/ppl/kernel/llm/cuda/pmx/i8i8/quantize.h:128-141.
//
//   z        = input + skip                      (fp16 add; skip may be null)          -> skip_out
//   r        = rsqrt(mean(z^2) + eps)
//   scale    = max(max(eps, max_k |z_k * w_k|) * r / 127, 1e-7)                        -> output_scale = fp16(scale * up_scale)
//   q_k      = clamp(round_half_away(((z_k * w_k) * r) * (1 / scale)), -127, 127)      -> output (int8)
//
// One CTA per row; the row (after the skip add) stays in registers between the statistics pass and
// the quantize pass, so HBM sees each input element once.  The sum of squares is accumulated in
// fp32 in this kernel's own order (per-thread chain, warp shuffles, cross-warp), which differs from
// the reference's CUB order; results agree to the last bit of the scale in almost all rows and to
// +-1 in the rare int8 value that sits on a rounding boundary.
#include "common.cuh"

namespace pplb200 {

namespace {

constexpr int RTPB = 256;

__device__ __forceinline__ uint4 ldg16(const void* p) { return *reinterpret_cast<const uint4*>(p); }

template <int UNITS>
__global__ void __launch_bounds__(RTPB)
skip_rmsnorm_quantize_kernel(const half* __restrict__ input, const half* __restrict__ weight, const half* __restrict__ skip,
                             float eps, int64_t batch, int64_t dim, float up_scale, int32_t layout,
                             half* __restrict__ skip_out, half* __restrict__ scale_out, int8_t* __restrict__ q) {
    __shared__ float red_sum[RTPB / 32];
    __shared__ float red_max[RTPB / 32];
    const int64_t row = blockIdx.x;
    const int units = (int)(dim >> 4);
    const half* in_row = input + row * dim;

    // ---- load, skip add, statistics
    __half2 z[UNITS][8];
    float sumsq = 0.0f;
    float amax = eps; // the reference seeds the running maximum with eps (rms_norm.cu:58)
#pragma unroll
    for (int u = 0; u < UNITS; ++u) {
        const int unit = u * blockDim.x + threadIdx.x;
        if (unit < units) {
            const int64_t off = (int64_t)unit << 4;
            uint4 a[2] = {ldg16(in_row + off), ldg16(in_row + off + 8)};
            __half2* h = reinterpret_cast<__half2*>(a);
            if (skip != nullptr) {
                uint4 s[2] = {ldg16(skip + row * dim + off), ldg16(skip + row * dim + off + 8)};
                const __half2* sh = reinterpret_cast<const __half2*>(s);
#pragma unroll
                for (int i = 0; i < 8; ++i) h[i] = __hadd2(h[i], sh[i]);
            }
            *reinterpret_cast<uint4*>(skip_out + row * dim + off) = a[0];
            *reinterpret_cast<uint4*>(skip_out + row * dim + off + 8) = a[1];
            uint4 wv[2] = {ldg16(weight + off), ldg16(weight + off + 8)};
            const __half2* wh = reinterpret_cast<const __half2*>(wv);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                z[u][i] = h[i];
                const float2 x = __half22float2(h[i]);
                const float2 w = __half22float2(wh[i]);
                sumsq = fmaf(x.x, x.x, sumsq);
                sumsq = fmaf(x.y, x.y, sumsq);
                amax = fmaxf(amax, fabsf(__fmul_rn(x.x, w.x)));
                amax = fmaxf(amax, fabsf(__fmul_rn(x.y, w.y)));
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) z[u][i] = __float2half2_rn(0.0f);
        }
    }
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) {
        sumsq += __shfl_xor_sync(0xffffffffu, sumsq, m);
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    if (lane == 0) { red_sum[warp] = sumsq; red_max[warp] = amax; }
    __syncthreads();
    float tot = red_sum[0], gmax = red_max[0];
    for (int w = 1; w < nwarps; ++w) { tot += red_sum[w]; gmax = fmaxf(gmax, red_max[w]); }

    const float mean = __fmul_rn(tot, __fdiv_rn(1.0f, (float)dim));
    const float r = rsqrtf(mean + eps);
    const float scale = fmaxf(__fdiv_rn(__fmul_rn(gmax, r), 127.0f), 1e-7f);
    const float inv_scale = __fdiv_rn(1.0f, scale);
    if (threadIdx.x == 0) scale_out[row] = __float2half_rn(scale * up_scale);

    // ---- quantize
#pragma unroll
    for (int u = 0; u < UNITS; ++u) {
        const int unit = u * blockDim.x + threadIdx.x;
        if (unit < units) {
            const int64_t off = (int64_t)unit << 4;
            uint4 wv[2] = {ldg16(weight + off), ldg16(weight + off + 8)};
            const __half2* wh = reinterpret_cast<const __half2*>(wv);
            int qi[16];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 x = __half22float2(z[u][i]);
                const float2 w = __half22float2(wh[i]);
                const float v0 = __fmul_rn(__fmul_rn(__fmul_rn(x.x, w.x), r), inv_scale);
                const float v1 = __fmul_rn(__fmul_rn(__fmul_rn(x.y, w.y), r), inv_scale);
                int q0 = (int)roundf(v0), q1 = (int)roundf(v1); // round half away from zero (quant_utils.h:86)
                qi[2 * i] = q0 > 127 ? 127 : (q0 < -127 ? -127 : q0);
                qi[2 * i + 1] = q1 > 127 ? 127 : (q1 < -127 ? -127 : q1);
            }
            uint4 o;
            uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                ow[i] = (uint32_t)(qi[4 * i] & 0xff) | ((uint32_t)(qi[4 * i + 1] & 0xff) << 8) |
                        ((uint32_t)(qi[4 * i + 2] & 0xff) << 16) | ((uint32_t)(qi[4 * i + 3] & 0xff) << 24);
            *reinterpret_cast<uint4*>(q + layout_offset(layout, batch, dim, row, off)) = o;
        }
    }
}

} // namespace

int32_t launch_skip_rmsnorm_quantize(cudaStream_t stream, const half* input, const half* weight, const half* skip,
                                     float eps, int64_t batch, int64_t dim, float up_scale, int32_t layout,
                                     half* skip_out, half* scale_out, int8_t* q) {
    if (batch == 0 || dim == 0) return RC_SUCCESS;
    const int64_t units = dim >> 4;
    if (units > RTPB * 8) return fail(RC_UNSUPPORTED, "normalize_shape %lld beyond %d", (long long)dim, RTPB * 8 * 16);
    const int per = (int)((units + RTPB - 1) / RTPB);
    const int bucket = per <= 1 ? 1 : per <= 2 ? 2 : per <= 4 ? 4 : 8;
    int threads = (int)((units + bucket - 1) / bucket);
    threads = (threads + 31) / 32 * 32;
    if (threads > RTPB) threads = RTPB;
    const dim3 grid((unsigned)batch), block(threads);
    switch (bucket) {
    case 1: skip_rmsnorm_quantize_kernel<1><<<grid, block, 0, stream>>>(input, weight, skip, eps, batch, dim, up_scale, layout, skip_out, scale_out, q); break;
    case 2: skip_rmsnorm_quantize_kernel<2><<<grid, block, 0, stream>>>(input, weight, skip, eps, batch, dim, up_scale, layout, skip_out, scale_out, q); break;
    case 4: skip_rmsnorm_quantize_kernel<4><<<grid, block, 0, stream>>>(input, weight, skip, eps, batch, dim, up_scale, layout, skip_out, scale_out, q); break;
    default: skip_rmsnorm_quantize_kernel<8><<<grid, block, 0, stream>>>(input, weight, skip, eps, batch, dim, up_scale, layout, skip_out, scale_out, q); break;
    }
    return check_launch("skip_rmsnorm_quantize");
}

} // namespace pplb200
