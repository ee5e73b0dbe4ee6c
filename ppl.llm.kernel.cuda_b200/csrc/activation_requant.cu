// Consumers of the raw int32 GEMM output (column_parallel_linear with gather_output = false):
//   dequantize + split into three tensors            (fused QKV projection)
//   dequantize + SiLU [x gate]  [+ re-quantize]      (separate gate / up projections)
//   dequantize + SwiGLU          + re-quantize       (fused gate+up projection: input = [x | gate])
// Reference: src/ppl/kernel/llm/cuda/pmx/i8i8/split.cu:44-169, silu.cu:44-199, swiglu.cu:42-185;
// declarations include/ppl/kernel/llm/cuda/pmx/i8i8/quantize.h:57-126.
//
// Arithmetic follows the reference kernels operation by operation (three separately rounded
// products for the dequant, __expf, IEEE division, row maximum of the fp32 result BEFORE it is
// rounded to fp16, quotient taken from the fp16-rounded value), so results are bit-identical to
// them.  One CTA per row; the activated row stays in registers between the maximum and the
// rounding pass instead of being re-read from the fp16 workspace (which is still written, as the
// reference does).
#include "common.cuh"

namespace pplb200 {

namespace {

constexpr int ATPB = 256;
enum : int { ACT_SILU = 0, ACT_SILU_GATED = 1, ACT_SWIGLU = 2 };

struct ActParams {
    const int32_t* input;
    const half* scale_batch; const half* scale_channel;
    const int32_t* gate; const half* gate_scale_batch; const half* gate_scale_channel; // ACT_SILU_GATED only
    int64_t batch, dim;
    float beta, up_scale, down_batch, down_channel;
    int32_t layout;
    half* workspace;  // fp16 activated values [batch, dim] in `layout` (may be null when not re-quantizing)
    int8_t* out_q;    // re-quantize: int8 [batch, dim] in `layout`
    half* out_h;      // no re-quantize: fp16 [batch, dim] in `layout`
    half* scale_out;  // re-quantize: fp16 [batch]
};

__device__ __forceinline__ float dq(int32_t v, half sc, float down_c, float bs) {
    return __fmul_rn(__fmul_rn(__fmul_rn((float)v, __half2float(sc)), down_c), bs);
}

__device__ __forceinline__ void load16_i32(const int32_t* p, int32_t (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int4 t = *reinterpret_cast<const int4*>(p + 4 * i);
        v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
}
__device__ __forceinline__ void load16_f16(const half* p, half (&v)[16]) {
    *reinterpret_cast<uint4*>(&v[0]) = *reinterpret_cast<const uint4*>(p);
    *reinterpret_cast<uint4*>(&v[8]) = *reinterpret_cast<const uint4*>(p + 8);
}

template <int UNITS, int KIND, bool REQUANT>
__global__ void __launch_bounds__(ATPB)
activation_rows_kernel(const ActParams p) {
    __shared__ float red[ATPB / 32];
    const int64_t row = blockIdx.x;
    const int units = (int)(p.dim >> 4);
    const int64_t in_cols = KIND == ACT_SWIGLU ? 2 * p.dim : p.dim;
    const float bs = __fmul_rn(__half2float(p.scale_batch[row]), p.down_batch);
    float gs = 0.0f;
    if (KIND == ACT_SILU_GATED) gs = __fmul_rn(__half2float(p.gate_scale_batch[row]), p.down_batch);

    half res[UNITS][16];
    float amax = 0.0f;
#pragma unroll
    for (int u = 0; u < UNITS; ++u) {
        const int unit = u * blockDim.x + threadIdx.x;
        if (unit < units) {
            const int64_t col = (int64_t)unit << 4;
            int32_t x[16]; half sc[16];
            load16_i32(p.input + layout_offset(p.layout, p.batch, in_cols, row, col), x);
            load16_f16(p.scale_channel + col, sc);
            int32_t g[16]; half gsc[16];
            if (KIND == ACT_SWIGLU) {
                load16_i32(p.input + layout_offset(p.layout, p.batch, in_cols, row, col + p.dim), g);
                load16_f16(p.scale_channel + col + p.dim, gsc);
            } else if (KIND == ACT_SILU_GATED) {
                load16_i32(p.gate + layout_offset(p.layout, p.batch, p.dim, row, col), g);
                load16_f16(p.gate_scale_channel + col, gsc);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float v = dq(x[i], sc[i], p.down_channel, bs);
                if (KIND == ACT_SWIGLU) {
                    const float gate = dq(g[i], gsc[i], p.down_channel, bs);
                    v = __fmul_rn(__fdiv_rn(v, __fadd_rn(1.0f, __expf(__fmul_rn(-v, p.beta)))), gate);
                } else {
                    v = __fdiv_rn(v, __fadd_rn(1.0f, __expf(-v)));
                    if (KIND == ACT_SILU_GATED) v = __fmul_rn(v, dq(g[i], gsc[i], p.down_channel, gs));
                }
                res[u][i] = __float2half_rn(v);
                amax = fmaxf(fabsf(v), amax);
            }
            half* dst = REQUANT ? p.workspace : p.out_h;
            if (dst != nullptr) {
                const int64_t off = layout_offset(p.layout, p.batch, p.dim, row, col);
                *reinterpret_cast<uint4*>(dst + off) = *reinterpret_cast<const uint4*>(&res[u][0]);
                *reinterpret_cast<uint4*>(dst + off + 8) = *reinterpret_cast<const uint4*>(&res[u][8]);
            }
        }
    }
    if (!REQUANT) return;

#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    if (lane == 0) red[warp] = amax;
    __syncthreads();
    amax = red[0];
    for (int w = 1; w < nwarps; ++w) amax = fmaxf(amax, red[w]);
    const float scale = fmaxf(__fdiv_rn(amax, 127.0f), 1e-7f);
    if (threadIdx.x == 0) p.scale_out[row] = __float2half_rn(scale * p.up_scale);

#pragma unroll
    for (int u = 0; u < UNITS; ++u) {
        const int unit = u * blockDim.x + threadIdx.x;
        if (unit < units) {
            uint4 o;
            uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t w4 = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int qv = __float2int_rn(__fdiv_rn(__half2float(res[u][4 * i + j]), scale));
                    w4 |= (uint32_t)(qv & 0xff) << (8 * j);
                }
                ow[i] = w4;
            }
            *reinterpret_cast<uint4*>(p.out_q + layout_offset(p.layout, p.batch, p.dim, row, (int64_t)unit << 4)) = o;
        }
    }
}

template <int KIND, bool REQUANT>
int32_t launch_act(cudaStream_t stream, const ActParams& p) {
    const int64_t units = p.dim >> 4;
    if (units > ATPB * 8) return fail(RC_UNSUPPORTED, "quant_dim %lld beyond %d", (long long)p.dim, ATPB * 8 * 16);
    const int per = (int)((units + ATPB - 1) / ATPB);
    const int bucket = per <= 1 ? 1 : per <= 2 ? 2 : per <= 4 ? 4 : 8;
    int threads = (int)((units + bucket - 1) / bucket);
    threads = (threads + 31) / 32 * 32;
    if (threads > ATPB) threads = ATPB;
    const dim3 grid((unsigned)p.batch), block(threads);
    switch (bucket) {
    case 1: activation_rows_kernel<1, KIND, REQUANT><<<grid, block, 0, stream>>>(p); break;
    case 2: activation_rows_kernel<2, KIND, REQUANT><<<grid, block, 0, stream>>>(p); break;
    case 4: activation_rows_kernel<4, KIND, REQUANT><<<grid, block, 0, stream>>>(p); break;
    default: activation_rows_kernel<8, KIND, REQUANT><<<grid, block, 0, stream>>>(p); break;
    }
    return check_launch("activation");
}

// dequantize (+bias) and scatter the columns into three row-major outputs; 4 columns per thread
__global__ void __launch_bounds__(256)
dequantize_split3_kernel(const int32_t* __restrict__ acc, const half* __restrict__ bias, const half* __restrict__ scale_m,
                         const half* __restrict__ scale_n, int64_t batch, int64_t dim, int64_t d0, int64_t d1, int64_t d2,
                         float down_m, float down_n, int32_t layout, half* __restrict__ o0, half* __restrict__ o1,
                         half* __restrict__ o2) {
    const int64_t chunks = dim >> 2, total = batch * chunks;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / chunks, n = (i - m * chunks) << 2;
        const float bs = __fmul_rn(__half2float(scale_m[m]), down_m);
        uint2 ov;
        half* o = reinterpret_cast<half*>(&ov);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            o[j] = __float2half_rn(dq(acc[layout_offset(layout, batch, dim, m, n + j)], scale_n[n + j], down_n, bs));
            if (bias != nullptr) o[j] = __hadd(o[j], bias[n + j]);
        }
        half* dst = nullptr; // the reference routes a 4-column group by its first column (split.cu:73-79)
        if (n < d0) dst = o0 + m * d0 + n;
        else if (n < d0 + d1) dst = o1 + m * d1 + (n - d0);
        else if (n < d0 + d1 + d2) dst = o2 + m * d2 + (n - d0 - d1);
        if (dst != nullptr) *reinterpret_cast<uint2*>(dst) = ov;
    }
}

int32_t check_act_common(const void* input, const void* sb, const void* sc, int64_t batch, int64_t dim, int32_t layout) {
    if (layout != LAYOUT_ROW_MAJOR && layout != LAYOUT_COL32 && layout != LAYOUT_COL32_2R_4R4)
        return fail(RC_UNSUPPORTED, "unsupported matrix layout: %d", layout);
    if (batch < 0 || dim < 0) return fail(RC_INVALID_VALUE, "negative extent");
    if (dim % 16) return fail(RC_INVALID_VALUE, "quant_dim must be a multiple of 16, got %lld", (long long)dim);
    if (layout != LAYOUT_ROW_MAJOR && dim % 32) return fail(RC_INVALID_VALUE, "COL32 layouts need quant_dim %% 32 == 0");
    if (layout == LAYOUT_COL32_2R_4R4 && batch % 32) return fail(RC_INVALID_VALUE, "COL32_2R_4R4 needs batch %% 32 == 0");
    if (batch > 0 && dim > 0 && (!input || !sb || !sc)) return fail(RC_INVALID_VALUE, "null pointer");
    if (!aligned16(input) || !aligned16(sc)) return fail(RC_INVALID_VALUE, "input and channel scales must be 16-byte aligned");
    if (batch > 0x7fffffffLL) return fail(RC_UNSUPPORTED, "batch beyond 2^31 - 1");
    return RC_SUCCESS;
}

} // namespace

int32_t act_silu(cudaStream_t stream, const void* input, const void* sb, const void* sc, const void* gate, const void* gsb,
                 const void* gsc, int64_t batch, int64_t dim, int32_t layout, float up, float down_b, float down_c,
                 void* workspace, void* out, void* scale_out, bool requant) {
    int32_t rc = check_act_common(input, sb, sc, batch, dim, layout);
    if (rc != RC_SUCCESS || batch == 0 || dim == 0) return rc;
    if (!out || (requant && !scale_out)) return fail(RC_INVALID_VALUE, "null output");
    if (gate && (!gsb || !gsc || !aligned16(gate) || !aligned16(gsc))) return fail(RC_INVALID_VALUE, "gate needs its scales (16-byte aligned)");
    if (!aligned16(out) || (workspace && !aligned16(workspace))) return fail(RC_INVALID_VALUE, "outputs must be 16-byte aligned");
    ActParams p = {};
    p.input = (const int32_t*)input; p.scale_batch = (const half*)sb; p.scale_channel = (const half*)sc;
    p.gate = (const int32_t*)gate; p.gate_scale_batch = (const half*)gsb; p.gate_scale_channel = (const half*)gsc;
    p.batch = batch; p.dim = dim; p.beta = 1.0f; p.up_scale = up; p.down_batch = down_b; p.down_channel = down_c;
    p.layout = layout; p.workspace = (half*)workspace; p.scale_out = (half*)scale_out;
    if (requant) p.out_q = (int8_t*)out; else p.out_h = (half*)out;
    if (requant) return gate ? launch_act<ACT_SILU_GATED, true>(stream, p) : launch_act<ACT_SILU, true>(stream, p);
    return gate ? launch_act<ACT_SILU_GATED, false>(stream, p) : launch_act<ACT_SILU, false>(stream, p);
}

int32_t act_swiglu(cudaStream_t stream, const void* input, const void* sb, const void* sc, int64_t batch, int64_t dim,
                   float beta, int32_t layout, float up, float down_b, float down_c, void* workspace, void* out,
                   void* scale_out) {
    int32_t rc = check_act_common(input, sb, sc, batch, dim, layout);
    if (rc != RC_SUCCESS || batch == 0 || dim == 0) return rc;
    if (!out || !scale_out) return fail(RC_INVALID_VALUE, "null output");
    if (!aligned16(out) || (workspace && !aligned16(workspace))) return fail(RC_INVALID_VALUE, "outputs must be 16-byte aligned");
    ActParams p = {};
    p.input = (const int32_t*)input; p.scale_batch = (const half*)sb; p.scale_channel = (const half*)sc;
    p.batch = batch; p.dim = dim; p.beta = beta; p.up_scale = up; p.down_batch = down_b; p.down_channel = down_c;
    p.layout = layout; p.workspace = (half*)workspace; p.out_q = (int8_t*)out; p.scale_out = (half*)scale_out;
    return launch_act<ACT_SWIGLU, true>(stream, p);
}

int32_t dequantize_split3(cudaStream_t stream, const void* acc, const void* bias, const void* sm, const void* sn,
                          int64_t batch, int64_t dim, int64_t d0, int64_t d1, int64_t d2, float down_m, float down_n,
                          int32_t layout, void* o0, void* o1, void* o2) {
    if (dim % 4 != 0) return fail(RC_INVALID_VALUE, "channel must be aligned with 4, but channel = %lld", (long long)dim);
    if (layout < LAYOUT_ROW_MAJOR || layout > LAYOUT_COL4_4R2_8C) return fail(RC_UNSUPPORTED, "unsupported matrix layout: %d", layout);
    if (batch < 0 || dim < 0 || d0 < 0 || d1 < 0 || d2 < 0) return fail(RC_INVALID_VALUE, "negative extent");
    if (d0 % 4 || d1 % 4 || d2 % 4) return fail(RC_INVALID_VALUE, "split sizes must be multiples of 4");
    if (batch == 0 || dim == 0) return RC_SUCCESS;
    if (!acc || !sm || !sn || (d0 && !o0) || (d1 && !o1) || (d2 && !o2)) return fail(RC_INVALID_VALUE, "null pointer");
    int64_t blocks = (batch * (dim >> 2) + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    dequantize_split3_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const int32_t*)acc, (const half*)bias, (const half*)sm,
                                                                   (const half*)sn, batch, dim, d0, d1, d2, down_m, down_n, layout,
                                                                   (half*)o0, (half*)o1, (half*)o2);
    return check_launch("dequantize_split3");
}

} // namespace pplb200
