// Per-token fp16 -> int8 quantizer, int32 -> fp16 dequantizer and the [w, M, n] -> [M, w, n]
// transpose of the tensor-parallel gather, for sm_100a.
//
// Semantics follow the reference kernels bit for bit:
//   quantizer   src/ppl/kernel/llm/cuda/pmx/i8i8/quantize.cu:27-80
//   dequantizer src/ppl/kernel/llm/cuda/pmx/i8i8/quantize.cu:126-169
// but the quantizer reads each row from HBM once (the row lives in registers between the
// absmax pass and the rounding pass) instead of twice.
#include "common.cuh"
#include "quant_device.cuh"

namespace pplb200 {

namespace {

using namespace qdev;

__device__ __forceinline__ void pdl_wait_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// One CTA per row.  A "unit" is 16 consecutive halves (two 128-bit loads, one 128-bit store).
// Thread t owns units t, t + blockDim.x, ... (UNITS of them), kept in registers.
template <int UNITS>
__global__ void __launch_bounds__(QTPB, UNITS <= 2 ? 5 : 1)
quantize_rows_kernel(const half* __restrict__ in, int64_t batch, int64_t dim, float up_scale, int32_t layout,
                     int8_t* __restrict__ q, half* __restrict__ scale_out, const uint32_t* __restrict__ given_absmax_bits,
                     uint32_t* __restrict__ zero_absmax_bits) {
    __shared__ float red[QTPB / 32];
    const int64_t row = blockIdx.x;
    const int units = (int)(dim >> 4);
    const uint4* src = reinterpret_cast<const uint4*>(in + row * dim);
    // With a precomputed row maximum the row may be split over blockIdx.y; otherwise gridDim.y == 1.
    const int unit_base = blockIdx.y * blockDim.x * UNITS;

    pdl_launch_dependents(); // a dependent kernel may start its own preamble now
    pdl_wait_prior_grid();   // no-op unless launched as a programmatic dependent

    uint4 v[UNITS][2];
#pragma unroll
    for (int u = 0; u < UNITS; ++u) {
        const int unit = unit_base + u * blockDim.x + threadIdx.x;
        if (unit < units) {
            v[u][0] = ldg_stream(src + 2 * unit);
            v[u][1] = ldg_stream(src + 2 * unit + 1);
        } else {
            v[u][0] = make_uint4(0, 0, 0, 0);
            v[u][1] = make_uint4(0, 0, 0, 0);
        }
    }

    // max |x| taken in fp16 (exact: max commutes with the widening conversion)
    QuantRow qr;
    if (given_absmax_bits == nullptr) {
        bool saw_nan, any_nan;
        float amax = absmax_halves(reinterpret_cast<const __half2*>(&v[0][0]), UNITS * 8, saw_nan);
        amax = block_max_any(amax, saw_nan, red, blockDim.x >> 5, any_nan);
        qr = make_quant_row(amax, any_nan);
    } else {
        qr = make_quant_row(__uint_as_float(given_absmax_bits[row]), false);
    }
    const float scale = qr.scale;

#pragma unroll
    for (int u = 0; u < UNITS; ++u) {
        const int unit = unit_base + u * blockDim.x + threadIdx.x;
        if (unit < units) {
            const uint4 o = given_absmax_bits == nullptr ? quant16<false>(reinterpret_cast<const __half2*>(&v[u][0]), qr)
                                                         : quant16<true>(reinterpret_cast<const __half2*>(&v[u][0]), qr);
            const int64_t off = layout_offset(layout, batch, dim, row, (int64_t)unit << 4);
            *reinterpret_cast<uint4*>(q + off) = o;
        }
    }
    if (threadIdx.x == 0 && blockIdx.y == 0) {
        scale_out[row] = __float2half_rn(scale * up_scale);
        if (zero_absmax_bits != nullptr) zero_absmax_bits[row] = 0u;
    }
}

// Rows too long for the register-resident kernel: classic two-pass (second read hits L2 for
// any realistic row length).
__global__ void __launch_bounds__(QTPB)
quantize_rows_twopass_kernel(const half* __restrict__ in, int64_t batch, int64_t dim, float up_scale, int32_t layout,
                             int8_t* __restrict__ q, half* __restrict__ scale_out,
                             const uint32_t* __restrict__ given_absmax_bits, uint32_t* __restrict__ zero_absmax_bits) {
    __shared__ float red[QTPB / 32];
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const int64_t row = blockIdx.x;
    const int64_t units = dim >> 4;
    const uint4* src = reinterpret_cast<const uint4*>(in + row * dim);
    float amax;
    if (given_absmax_bits == nullptr) {
        __half2 m2 = __float2half2_rn(0.0f);
        for (int64_t unit = threadIdx.x; unit < units; unit += blockDim.x) {
            uint4 a[2] = {src[2 * unit], src[2 * unit + 1]};
            const __half2* h = reinterpret_cast<const __half2*>(a);
#pragma unroll
            for (int i = 0; i < 8; ++i) m2 = __hmax2(m2, __habs2(h[i]));
        }
        amax = block_max(fmaxf(__low2float(m2), __high2float(m2)), red, blockDim.x >> 5);
    } else {
        amax = __uint_as_float(given_absmax_bits[row]);
    }
    const QuantRow qr = make_quant_row(amax, false);
    const float scale = qr.scale;
    for (int64_t unit = threadIdx.x; unit < units; unit += blockDim.x) {
        uint4 a[2] = {src[2 * unit], src[2 * unit + 1]};
        const uint4 o = quant16<true>(reinterpret_cast<const __half2*>(a), qr); // NaNs were dropped above: looked for per group
        *reinterpret_cast<uint4*>(q + layout_offset(layout, batch, dim, row, unit << 4)) = o;
    }
    if (threadIdx.x == 0) {
        scale_out[row] = __float2half_rn(scale * up_scale);
        if (zero_absmax_bits != nullptr) zero_absmax_bits[row] = 0u;
    }
}

// ---- dequantize ------------------------------------------------------------------------------

__device__ __forceinline__ half dequant_one(int32_t acc, half sn, float down_n, float batch_scale) {
    // three separately rounded fp32 products, left to right (quantize.cu:157)
    float t = __fmul_rn((float)acc, __half2float(sn));
    t = __fmul_rn(t, down_n);
    t = __fmul_rn(t, batch_scale);
    return __float2half_rn(t);
}

// Row-major int32 in, 8 outputs per thread (N % 8 == 0).
__global__ void __launch_bounds__(256)
dequantize_rowmajor8_kernel(const int32_t* __restrict__ acc, const half* __restrict__ bias,
                            const half* __restrict__ scale_m, const half* __restrict__ scale_n,
                            int64_t batch, int64_t dim, float down_m, float down_n, half* __restrict__ out) {
    const int64_t chunks_per_row = dim >> 3;
    const int64_t total = batch * chunks_per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / chunks_per_row;
        const int64_t n = (i - m * chunks_per_row) << 3;
        const float bs = __fmul_rn(__half2float(scale_m[m]), down_m);
        const int4 a0 = *reinterpret_cast<const int4*>(acc + m * dim + n);
        const int4 a1 = *reinterpret_cast<const int4*>(acc + m * dim + n + 4);
        const uint4 snv = *reinterpret_cast<const uint4*>(scale_n + n);
        const half* sn = reinterpret_cast<const half*>(&snv);
        const int32_t a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        uint4 ov;
        half* o = reinterpret_cast<half*>(&ov);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = dequant_one(a[j], sn[j], down_n, bs);
        if (bias != nullptr) {
            const uint4 bv = *reinterpret_cast<const uint4*>(bias + n);
            const half* b = reinterpret_cast<const half*>(&bv);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = __hadd(o[j], b[j]);
        }
        *reinterpret_cast<uint4*>(out + m * dim + n) = ov;
    }
}

// Any layout / N % 4 == 0: 4 outputs per thread, per-element gather.
__global__ void __launch_bounds__(256)
dequantize_generic4_kernel(const int32_t* __restrict__ acc, const half* __restrict__ bias,
                           const half* __restrict__ scale_m, const half* __restrict__ scale_n,
                           int64_t batch, int64_t dim, float down_m, float down_n, int32_t layout,
                           half* __restrict__ out) {
    const int64_t chunks_per_row = dim >> 2;
    const int64_t total = batch * chunks_per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / chunks_per_row;
        const int64_t n = (i - m * chunks_per_row) << 2;
        const float bs = __fmul_rn(__half2float(scale_m[m]), down_m);
        uint2 ov;
        half* o = reinterpret_cast<half*>(&ov);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int32_t a = acc[layout_offset(layout, batch, dim, m, n + j)];
            o[j] = dequant_one(a, scale_n[n + j], down_n, bs);
            if (bias != nullptr) o[j] = __hadd(o[j], bias[n + j]);
        }
        *reinterpret_cast<uint2*>(out + m * dim + n) = ov;
    }
}

// [d0, d1, d2] -> [d1, d0, d2] on fp16, 8 halves per thread when d2 % 8 == 0.
template <typename VEC>
__global__ void __launch_bounds__(256)
transpose01_kernel(const VEC* __restrict__ in, int64_t d0, int64_t d1, int64_t d2v, VEC* __restrict__ out) {
    const int64_t total = d0 * d1 * d2v;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t c = i % d2v, b = (i / d2v) % d1, a = i / (d2v * d1);
        out[(b * d0 + a) * d2v + c] = in[i];
    }
}

// Element-wise change of storage order of a [rows, cols] matrix, four consecutive columns (which every
// layout but COL_MAJOR keeps contiguous) per item.  VEC = uint32_t for int8 elements, uint4 for int32.
template <typename VEC>
__global__ void __launch_bounds__(256)
relayout4_kernel(const VEC* __restrict__ src, int32_t src_layout, VEC* __restrict__ dst, int32_t dst_layout, int64_t rows,
                 int64_t cols) {
    const int64_t quads_per_row = cols >> 2;
    const int64_t total = rows * quads_per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        // walk the DESTINATION in storage order where it is row-major (the common direction: legacy -> row-major)
        const int64_t r = i / quads_per_row, c = (i - r * quads_per_row) << 2;
        dst[layout_offset(dst_layout, rows, cols, r, c) >> 2] = src[layout_offset(src_layout, rows, cols, r, c) >> 2];
    }
}

int grid_for(int64_t work_items, int tpb) {
    int64_t blocks = (work_items + tpb - 1) / tpb;
    const int64_t cap = 148 * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

template <typename... Args>
cudaError_t launch_ex(void (*kernel)(Args...), dim3 grid, dim3 block, cudaStream_t stream, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

} // namespace

int32_t launch_quantize(cudaStream_t stream, const half* in, int64_t batch, int64_t dim, float up_scale,
                        int32_t layout, int8_t* q, half* scale, const uint32_t* given_absmax_bits,
                        uint32_t* zero_absmax_bits, bool pdl) {
    if (batch == 0 || dim == 0) return RC_SUCCESS;
    const int64_t units = dim >> 4;
    cudaError_t e;
    if (given_absmax_bits != nullptr && units <= (int64_t)QTPB * 65535) {
        // the row maximum is known: no reduction, so a row is spread over as many CTAs as it has
        // 256-unit chunks (more loads in flight when there are few rows)
        int threads = (int)(units < QTPB ? (units + 31) / 32 * 32 : QTPB);
        const dim3 grid((unsigned)batch, (unsigned)((units + threads - 1) / threads), 1);
        e = launch_ex(quantize_rows_kernel<1>, grid, dim3(threads), stream, pdl, in, batch, dim, up_scale, layout, q, scale,
                      given_absmax_bits, zero_absmax_bits);
    } else if (units <= QTPB * 8) {
        // threads: enough to give every thread the same small number of units
        int per = (int)((units + QTPB - 1) / QTPB);
        int bucket = per <= 1 ? 1 : per <= 2 ? 2 : per <= 4 ? 4 : 8;
        // Rows of 8192 halves and more: four units (128 bytes of loads) per thread and half as many threads keep more
        // bytes in flight per SM than two units per thread do (measured 40.4 vs 41.8 us on 8192 x 8192).
        if (bucket == 2 && units >= 512) bucket = 4;
        int threads = (int)((units + bucket - 1) / bucket);
        threads = (threads + 31) / 32 * 32;
        if (threads > QTPB) threads = QTPB;
        const dim3 grid((unsigned)batch, 1, 1), block(threads);
        switch (bucket) {
        case 1: e = launch_ex(quantize_rows_kernel<1>, grid, block, stream, pdl, in, batch, dim, up_scale, layout, q, scale, given_absmax_bits, zero_absmax_bits); break;
        case 2: e = launch_ex(quantize_rows_kernel<2>, grid, block, stream, pdl, in, batch, dim, up_scale, layout, q, scale, given_absmax_bits, zero_absmax_bits); break;
        case 4: e = launch_ex(quantize_rows_kernel<4>, grid, block, stream, pdl, in, batch, dim, up_scale, layout, q, scale, given_absmax_bits, zero_absmax_bits); break;
        default: e = launch_ex(quantize_rows_kernel<8>, grid, block, stream, pdl, in, batch, dim, up_scale, layout, q, scale, given_absmax_bits, zero_absmax_bits); break;
        }
    } else {
        e = launch_ex(quantize_rows_twopass_kernel, dim3((unsigned)batch), dim3(QTPB), stream, pdl, in, batch, dim, up_scale, layout, q, scale,
                      given_absmax_bits, zero_absmax_bits);
    }
    if (e != cudaSuccess) return fail(RC_DEVICE_RUNTIME_ERROR, "quantize launch failed: %s", cudaGetErrorString(e));
    return RC_SUCCESS;
}

int32_t launch_dequantize(cudaStream_t stream, const int32_t* acc, const half* bias, const half* scale_m,
                          const half* scale_n, int64_t batch, int64_t dim, float down_m, float down_n,
                          int32_t layout, half* out) {
    if (batch == 0 || dim == 0) return RC_SUCCESS;
    const bool vec8 = layout == LAYOUT_ROW_MAJOR && (dim % 8 == 0) && aligned16(acc) && aligned16(out) &&
                      aligned16(scale_n) && (bias == nullptr || aligned16(bias));
    if (vec8) {
        dequantize_rowmajor8_kernel<<<grid_for(batch * (dim >> 3), 256), 256, 0, stream>>>(
            acc, bias, scale_m, scale_n, batch, dim, down_m, down_n, out);
    } else {
        dequantize_generic4_kernel<<<grid_for(batch * (dim >> 2), 256), 256, 0, stream>>>(
            acc, bias, scale_m, scale_n, batch, dim, down_m, down_n, layout, out);
    }
    return check_launch("dequantize");
}

int32_t launch_relayout(cudaStream_t stream, const void* src, int32_t src_layout, void* dst, int32_t dst_layout,
                        int64_t rows, int64_t cols, int32_t elem_bytes) {
    if (rows * cols == 0) return RC_SUCCESS;
    const int grid = grid_for(rows * (cols >> 2), 256);
    if (elem_bytes == 1)
        relayout4_kernel<uint32_t><<<grid, 256, 0, stream>>>((const uint32_t*)src, src_layout, (uint32_t*)dst, dst_layout, rows, cols);
    else
        relayout4_kernel<uint4><<<grid, 256, 0, stream>>>((const uint4*)src, src_layout, (uint4*)dst, dst_layout, rows, cols);
    return check_launch("relayout");
}

int32_t launch_transpose01_f16(cudaStream_t stream, const half* in, int64_t d0, int64_t d1, int64_t d2, half* out) {
    if (d0 * d1 * d2 == 0) return RC_SUCCESS;
    if (d2 % 8 == 0 && aligned16(in) && aligned16(out)) {
        transpose01_kernel<uint4><<<grid_for(d0 * d1 * (d2 >> 3), 256), 256, 0, stream>>>(
            reinterpret_cast<const uint4*>(in), d0, d1, d2 >> 3, reinterpret_cast<uint4*>(out));
    } else {
        transpose01_kernel<uint16_t><<<grid_for(d0 * d1 * d2, 256), 256, 0, stream>>>(
            reinterpret_cast<const uint16_t*>(in), d0, d1, d2, reinterpret_cast<uint16_t*>(out));
    }
    return check_launch("transpose01");
}

} // namespace pplb200
