/*
 * TEST INFRASTRUCTURE ONLY -- see oracle.h.  Scalar host restatement of the
 * W8A8 (i8i8) linear path of OpenPPL/ppl.llm.kernel.cuda; the checker for the
 * CUDA kernels and the timed CPU baseline.  Never linked into the product.
 *
 * Build: gcc -O3 -march=x86-64-v3 -ffp-contract=off -fno-fast-math -fPIC -shared -pthread
 * (-ffp-contract=off matters: the reference's dequant is three separately
 *  rounded fp32 multiplies, and nothing here may be fused into an FMA).
 */
#include "oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ fp16 */

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint64_t f64_bits(double d) { uint64_t u; memcpy(&u, &d, 8); return u; }

/* Generic round-to-nearest-even narrowing of (sign, unbiased exponent e, 64-bit
 * significand sig with the leading one at bit 63) to binary16. */
static uint16_t pack_f16(uint32_t sign, int32_t e, uint64_t sig) {
    /* value = sig * 2^(e-63), sig in [2^63, 2^64) */
    if (e > 15) return (uint16_t)(sign | 0x7C00u);            /* overflow -> inf (rn) */
    int32_t shift;                                             /* bits to drop from sig */
    uint32_t exp_field;
    if (e >= -14) { shift = 63 - 10; exp_field = (uint32_t)(e + 15); }
    else          { shift = 63 - 10 + (-14 - e); exp_field = 0; }
    if (shift > 64) return (uint16_t)sign;                     /* far below half of the smallest subnormal */
    uint64_t kept, rem, half;
    if (shift == 64) { kept = 0; rem = sig; half = 1ull << 63; }
    else {
        kept = sig >> shift;
        rem  = sig & ((1ull << shift) - 1);
        half = 1ull << (shift - 1);
    }
    if (rem > half || (rem == half && (kept & 1))) kept += 1;
    /* kept holds [hidden bit +] 10 mantissa bits; a carry may bump the exponent, which the
     * plain integer addition below handles (also subnormal -> normal and normal -> inf). */
    uint32_t out;
    if (exp_field == 0) out = (uint32_t)kept;                                   /* subnormal or just became normal */
    else                out = ((exp_field - 1) << 10) + (uint32_t)kept;         /* kept includes the hidden bit (1<<10) */
    if (out >= 0x7C00u) out = 0x7C00u;
    return (uint16_t)(sign | out);
}

uint16_t orc_f32_to_f16(float f) {
    uint32_t u = f32_bits(f);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t ex = (u >> 23) & 0xFF;
    uint32_t man = u & 0x7FFFFFu;
    if (ex == 0xFF) return (uint16_t)(sign | (man ? 0x7FFFu : 0x7C00u)); /* NaN -> canonical, as cvt.rn.f16.f32 */
    if (ex == 0 && man == 0) return (uint16_t)sign;
    int32_t e; uint64_t sig;
    if (ex == 0) { /* fp32 subnormal: normalise */
        int lz = __builtin_clz(man) - 8; /* man < 2^23: zeros below the hidden-bit position */
        sig = (uint64_t)man << (40 + lz);
        e = -126 - lz;
    } else {
        sig = ((uint64_t)(man | 0x800000u)) << 40;
        e = (int32_t)ex - 127;
    }
    return pack_f16(sign, e, sig);
}

uint16_t orc_f64_to_f16(double d) {
    uint64_t u = f64_bits(d);
    uint32_t sign = (uint32_t)(u >> 48) & 0x8000u;
    uint32_t ex = (uint32_t)(u >> 52) & 0x7FF;
    uint64_t man = u & 0xFFFFFFFFFFFFFull;
    if (ex == 0x7FF) return (uint16_t)(sign | (man ? 0x7FFFu : 0x7C00u));
    if (ex == 0) return (uint16_t)sign; /* zero or fp64 subnormal: far below fp16 range */
    uint64_t sig = (man | (1ull << 52)) << 11;
    return pack_f16(sign, (int32_t)ex - 1023, sig);
}

float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t ex = (h >> 10) & 0x1F;
    uint32_t man = h & 0x3FFu;
    if (ex == 0x1F) return bits_f32(sign | 0x7F800000u | (man << 13));
    if (ex == 0) {
        if (man == 0) return bits_f32(sign);
        int lz = __builtin_clz(man) - 21; /* man < 2^10: shift that brings the top bit to bit 10 */
        man = (man << lz) & 0x3FFu;
        return bits_f32(sign | ((uint32_t)(113 - lz) << 23) | (man << 13));
    }
    return bits_f32(sign | ((ex + 112) << 23) | (man << 13));
}

/* The exact sum of two binary16 values fits a double, so converting that double
 * is a single rounding -- what the device's native half add does
 * (pmx/i8i8/quantize.cu:163, `local_out[i] + local_w[i]` on __half). */
uint16_t orc_f16_add(uint16_t a, uint16_t b) {
    double s = (double)orc_f16_to_f32(a) + (double)orc_f16_to_f32(b);
    return orc_f64_to_f16(s);
}

/* ------------------------------------------------------------------ layouts */

/* include/ppl/kernel/llm/cuda/common/matrix_layout.h:34-142 */
int64_t orc_layout_offset(int32_t layout, int64_t rows, int64_t cols, int64_t r, int64_t c) {
    switch (layout) {
    case ORC_LAYOUT_ROW_MAJOR: return r * cols + c;                       /* :46 */
    case ORC_LAYOUT_COL_MAJOR: return c * rows + r;                       /* :61 */
    case ORC_LAYOUT_COL32:     return (c / 32) * 32 * rows + r * 32 + c % 32; /* :77 */
    case ORC_LAYOUT_COL4_4R2_8C: {                                        /* :99-112 */
        int64_t panel = c / 32, cc = c % 32;
        int64_t in_panel = ((r / 8) * 8 + (r % 2) * 4 + cc / 8) * 32
                         + (((cc % 8) >= 4 ? 4 : 0) + (r % 8) / 2) * 4
                         + cc % 4;
        return panel * rows * 32 + in_panel;
    }
    case ORC_LAYOUT_COL32_2R_4R4: {                                       /* :132-141 */
        int64_t panel = c / 32, cc = c % 32, rt = r % 32;
        int64_t in_panel = (r / 32) * 1024 + ((((rt % 8) / 2) * 4 + rt / 8) * 2 + rt % 2) * 32 + cc;
        return panel * rows * 32 + in_panel;
    }
    default: return -1;
    }
}

/* ------------------------------------------------------------------ threads */

static int32_t g_threads = 1;
void orc_set_threads(int32_t n) { g_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }
int32_t orc_get_threads(void) { return g_threads; }

typedef void (*row_fn)(int64_t r0, int64_t r1, void* ctx);
typedef struct { row_fn fn; void* ctx; int64_t r0, r1; } job_t;
static void* job_main(void* p) { job_t* j = (job_t*)p; j->fn(j->r0, j->r1, j->ctx); return NULL; }

static void parallel_rows(int64_t r0, int64_t r1, row_fn fn, void* ctx) {
    int64_t n = r1 - r0;
    int32_t t = g_threads;
    if (t > n) t = (int32_t)(n > 0 ? n : 1);
    if (t <= 1) { fn(r0, r1, ctx); return; }
    pthread_t th[256]; job_t jobs[256];
    for (int32_t i = 0; i < t; ++i) {
        jobs[i].fn = fn; jobs[i].ctx = ctx;
        jobs[i].r0 = r0 + n * i / t; jobs[i].r1 = r0 + n * (i + 1) / t;
        pthread_create(&th[i], NULL, job_main, &jobs[i]);
    }
    for (int32_t i = 0; i < t; ++i) pthread_join(th[i], NULL);
}

/* ------------------------------------------------------------------ quantize */

/* __float2int_rn: round-to-nearest-even, NaN -> 0, saturating at the int32 range. */
static inline int32_t float2int_rn(float v) {
    if (v != v) return 0;
    if (v >= 2147483648.0f) return 2147483647;
    if (v <= -2147483648.0f) return (int32_t)0x80000000u;
    return (int32_t)nearbyintf(v); /* default rounding mode: to nearest even */
}

typedef struct {
    const uint16_t* x; int64_t batch, dim; float up; int32_t layout; int8_t* q; uint16_t* s;
} quant_ctx;

static void quant_rows(int64_t r0, int64_t r1, void* p) {
    quant_ctx* c = (quant_ctx*)p;
    for (int64_t r = r0; r < r1; ++r) {
        const uint16_t* row = c->x + r * c->dim;
        /* quantize.cu:46-57: running fmax(fabs(v), local_max) seeded with 0; fmax drops NaNs */
        float amax = 0.0f;
        for (int64_t k = 0; k < c->dim; ++k) amax = fmaxf(fabsf(orc_f16_to_f32(row[k])), amax);
        /* quantize.cu:58 -> quant_utils.h:119-125: max(range / 127, QTHRESHOLD=1e-7f) */
        float scale = fmaxf(amax / (float)127, 1e-7f);
        /* quantize.cu:63-75: q = (int8)__float2int_rn(v / scale), true IEEE division */
        for (int64_t k = 0; k < c->dim; ++k) {
            float v = orc_f16_to_f32(row[k]);
            c->q[orc_layout_offset(c->layout, c->batch, c->dim, r, k)] = (int8_t)float2int_rn(v / scale);
        }
        /* quantize.cu:77-79 */
        c->s[r] = orc_f32_to_f16(scale * c->up);
    }
}

int32_t orc_minmax_quantize_fp16(const uint16_t* x, int64_t batch, int64_t quant_dim, float up_scale,
                                 int32_t to_layout, int8_t* q, uint16_t* scale) {
    /* quantize.cu:94-121: ROW_MAJOR, COL_MAJOR, COL32, COL32_2R_4R4 are dispatched.  The kernel
     * stores 16 consecutive columns as 16 consecutive bytes at GetOffset(row, col0), which is
     * only a faithful element mapping where 16 aligned columns are contiguous: not COL_MAJOR. */
    if (to_layout != ORC_LAYOUT_ROW_MAJOR && to_layout != ORC_LAYOUT_COL32 &&
        to_layout != ORC_LAYOUT_COL32_2R_4R4)
        return 2;
    quant_ctx c = { x, batch, quant_dim, up_scale, to_layout, q, scale };
    parallel_rows(0, batch, quant_rows, &c);
    return 0;
}

/* ------------------------------------------------------------------ GEMM */

typedef struct {
    const int8_t* A; int64_t lda; const int8_t* B; int64_t ldb; int64_t N, K; int32_t* C; int64_t ldc; int64_t m_base;
} gemm_ctx;

static void gemm_rows(int64_t r0, int64_t r1, void* p) {
    gemm_ctx* g = (gemm_ctx*)p;
    for (int64_t m = r0; m < r1; ++m) {
        const int8_t* a = g->A + m * g->lda;
        int32_t* c = g->C + (m - g->m_base) * g->ldc;
        for (int64_t n = 0; n < g->N; ++n) {
            const int8_t* b = g->B + n * g->ldb;
            int32_t acc = 0;
            for (int64_t k = 0; k < g->K; ++k) acc += (int32_t)a[k] * (int32_t)b[k];
            c[n] = acc; /* alpha = 1, beta = 0: column_parallel_linear.cu:111-112 */
        }
    }
}

void orc_gemm_i8i8i32_rows(const int8_t* A, int64_t lda, const int8_t* B, int64_t ldb,
                           int64_t m0, int64_t m1, int64_t N, int64_t K, int32_t* C, int64_t ldc) {
    gemm_ctx g = { A, lda, B, ldb, N, K, C, ldc, m0 };
    parallel_rows(m0, m1, gemm_rows, &g);
}

void orc_gemm_i8i8i32(const int8_t* A, int64_t lda, const int8_t* B, int64_t ldb,
                      int64_t M, int64_t N, int64_t K, int32_t* C, int64_t ldc) {
    gemm_ctx g = { A, lda, B, ldb, N, K, C, ldc, 0 };
    parallel_rows(0, M, gemm_rows, &g);
}

/* ------------------------------------------------------------------ dequantize */

typedef struct {
    const int32_t* acc; const uint16_t *bias, *sm, *sn; int64_t batch, dim; float dm, dn; int32_t layout; uint16_t* out;
} deq_ctx;

static void deq_rows(int64_t r0, int64_t r1, void* p) {
    deq_ctx* d = (deq_ctx*)p;
    for (int64_t m = r0; m < r1; ++m) {
        /* quantize.cu:153 */
        float batch_scale = orc_f16_to_f32(d->sm[m]) * d->dm;
        for (int64_t n = 0; n < d->dim; ++n) {
            int32_t a = d->acc[orc_layout_offset(d->layout, d->batch, d->dim, m, n)];
            /* quantize.cu:157: ((float(acc) * float(scale_n)) * down_n) * batch_scale, each product rounded */
            float t = (float)a * orc_f16_to_f32(d->sn[n]);
            t = t * d->dn;
            t = t * batch_scale;
            uint16_t h = orc_f32_to_f16(t);
            /* quantize.cu:160-165: fp16 add of the bias */
            if (d->bias) h = orc_f16_add(h, d->bias[n]);
            d->out[m * d->dim + n] = h; /* quantize.cu:167: output is always row-major */
        }
    }
}

int32_t orc_minmax_dequantize_fp16(const int32_t* acc, const uint16_t* bias, const uint16_t* scale_m,
                                   const uint16_t* scale_n, int64_t batch, int64_t quant_dim,
                                   float down_m, float down_n, int32_t from_layout, uint16_t* out) {
    if (quant_dim % 4 != 0) return 4;                       /* quantize.cu:193-196 RC_INVALID_VALUE */
    if (from_layout < 0 || from_layout > 4) return 2;       /* quantize.cu:228-231 RC_UNSUPPORTED */
    deq_ctx d = { acc, bias, scale_m, scale_n, batch, quant_dim, down_m, down_n, from_layout, out };
    parallel_rows(0, batch, deq_rows, &d);
    return 0;
}

/* ------------------------------------------------------------------ whole path */

int32_t orc_w8a8_linear(const uint16_t* x, const int8_t* w, const uint16_t* scale_n, const uint16_t* bias,
                        int64_t M, int64_t N, int64_t K, float up_scale, float down_m, float down_n,
                        float requant_up_scale,
                        int8_t* xq, uint16_t* sm, int32_t* acc, uint16_t* y, int8_t* yq, uint16_t* yq_scale) {
    int8_t* xq_l = xq ? xq : (int8_t*)malloc((size_t)(M * K));
    uint16_t* sm_l = sm ? sm : (uint16_t*)malloc((size_t)M * 2);
    int32_t* acc_l = acc ? acc : (int32_t*)malloc((size_t)(M * N) * 4);
    int32_t rc = orc_minmax_quantize_fp16(x, M, K, up_scale, ORC_LAYOUT_ROW_MAJOR, xq_l, sm_l);
    if (rc == 0) {
        orc_gemm_i8i8i32(xq_l, K, w, K, M, N, K, acc_l, N);
        rc = orc_minmax_dequantize_fp16(acc_l, bias, sm_l, scale_n, M, N, down_m, down_n, ORC_LAYOUT_ROW_MAJOR, y);
    }
    if (rc == 0 && yq && yq_scale)
        rc = orc_minmax_quantize_fp16(y, M, N, requant_up_scale, ORC_LAYOUT_ROW_MAJOR, yq, yq_scale);
    if (!xq) free(xq_l);
    if (!sm) free(sm_l);
    if (!acc) free(acc_l);
    return rc;
}

void orc_sum_partials_i32(const int32_t* const* parts, int32_t nparts, int64_t count, int32_t* out) {
    for (int64_t i = 0; i < count; ++i) {
        uint32_t s = 0; /* wraparound two's-complement sum, like the device */
        for (int32_t p = 0; p < nparts; ++p) s += (uint32_t)parts[p][i];
        out[i] = (int32_t)s;
    }
}

/* ------------------------------------------------------------------ skip + RMSNorm + quantize */

typedef struct {
    const uint16_t *in, *w, *skip; float eps; int64_t batch, dim; float up; int32_t layout;
    uint16_t *skip_out, *scale; int8_t* q;
} rms_ctx;

static void rms_rows(int64_t r0, int64_t r1, void* p) {
    rms_ctx* c = (rms_ctx*)p;
    for (int64_t r = r0; r < r1; ++r) {
        const uint16_t* in = c->in + r * c->dim;
        uint16_t* z = c->skip_out + r * c->dim;
        double sumsq = 0.0;
        float amax = c->eps;                                                /* rms_norm.cu:58 */
        for (int64_t k = 0; k < c->dim; ++k) {
            z[k] = c->skip ? orc_f16_add(in[k], c->skip[r * c->dim + k]) : in[k];   /* :62-69 */
            float x = orc_f16_to_f32(z[k]), w = orc_f16_to_f32(c->w[k]);
            sumsq += (double)x * (double)x;                                 /* :76 */
            amax = fmaxf(amax, fabsf(x * w));                               /* :77 */
        }
        float mean = (float)sumsq * (1.0f / (float)c->dim);                 /* :86 */
        float rr = (float)(1.0 / sqrt((double)(mean + c->eps)));            /* :88 rsqrtf */
        float scale = fmaxf((amax * rr) / (float)127, 1e-7f);               /* :89, quant_utils.h:119-125 */
        c->scale[r] = orc_f32_to_f16(scale * c->up);                        /* :90 */
        float inv = 1.0f / scale;                                           /* quant_utils.h:84 */
        for (int64_t k = 0; k < c->dim; ++k) {
            float x = orc_f16_to_f32(z[k]), w = orc_f16_to_f32(c->w[k]);
            float v = ((x * w) * rr) * inv;                                 /* :97, quant_utils.h:84 */
            int32_t qi = (int32_t)roundf(v);                                /* quant_utils.h:86: half away from zero */
            qi = qi > 127 ? 127 : (qi < -127 ? -127 : qi);                  /* :87-88 */
            c->q[orc_layout_offset(c->layout, c->batch, c->dim, r, k)] = (int8_t)qi;
        }
    }
}

int32_t orc_skip_rmsnorm_minmax_quantize_fp16(const uint16_t* input, const uint16_t* weight, const uint16_t* skip,
                                              float eps, int64_t batch, int64_t dim, float up_scale, int32_t to_layout,
                                              uint16_t* skip_out, uint16_t* out_scale, int8_t* q) {
    if (to_layout != ORC_LAYOUT_ROW_MAJOR && to_layout != ORC_LAYOUT_COL32 && to_layout != ORC_LAYOUT_COL32_2R_4R4)
        return 2;
    rms_ctx c = { input, weight, skip, eps, batch, dim, up_scale, to_layout, skip_out, out_scale, q };
    parallel_rows(0, batch, rms_rows, &c);
    return 0;
}

/* ------------------------------------------------------------------ activation consumers */

int32_t orc_activation_requantize(int32_t kind, const int32_t* input, const uint16_t* scale_b, const uint16_t* scale_c,
                                  const int32_t* gate, const uint16_t* gate_scale_b, const uint16_t* gate_scale_c,
                                  int64_t batch, int64_t dim, float beta, float up_scale, float down_b, float down_c,
                                  uint16_t* workspace, int8_t* out_q, uint16_t* out_scale) {
    if (kind < 0 || kind > 2) return 2;
    const int64_t in_cols = kind == 2 ? 2 * dim : dim;
    for (int64_t r = 0; r < batch; ++r) {
        float bs = orc_f16_to_f32(scale_b[r]) * down_b;                                   /* silu.cu:68, swiglu.cu:67 */
        float gs = kind == 1 ? orc_f16_to_f32(gate_scale_b[r]) * down_b : 0.0f;           /* silu.cu:69 */
        float lmax = 0.0f;
        for (int64_t i = 0; i < dim; ++i) {
            float v = (float)input[r * in_cols + i] * orc_f16_to_f32(scale_c[i]);         /* silu.cu:95, swiglu.cu:92 */
            v = v * down_c; v = v * bs;
            if (kind == 2) {
                float g = (float)input[r * in_cols + dim + i] * orc_f16_to_f32(scale_c[dim + i]);
                g = g * down_c; g = g * bs;                                               /* swiglu.cu:93 */
                v = (v / (1.0f + expf(-v * beta))) * g;                                   /* swiglu.cu:96 */
            } else {
                v = v / (1.0f + expf(-v));                                                /* silu.cu:98 */
                if (kind == 1) {
                    float g = (float)gate[r * dim + i] * orc_f16_to_f32(gate_scale_c[i]); /* silu.cu:101 */
                    g = g * down_c; g = g * gs;
                    v = v * g;
                }
            }
            workspace[r * dim + i] = orc_f32_to_f16(v);                                   /* silu.cu:104 */
            lmax = fmaxf(fabsf(v), lmax);                                                 /* silu.cu:105 */
        }
        if (out_q && out_scale) {
            float scale = fmaxf(lmax / (float)127, 1e-7f);                                /* silu.cu:112 */
            out_scale[r] = orc_f32_to_f16(scale * up_scale);                              /* silu.cu:114 */
            for (int64_t i = 0; i < dim; ++i)                                             /* silu.cu:127 */
                out_q[r * dim + i] = (int8_t)float2int_rn(orc_f16_to_f32(workspace[r * dim + i]) / scale);
        }
    }
    return 0;
}

int32_t orc_dequantize_split3(const int32_t* acc, const uint16_t* bias, const uint16_t* scale_m, const uint16_t* scale_n,
                              int64_t batch, int64_t dim, int64_t d0, int64_t d1, int64_t d2, float down_m, float down_n,
                              uint16_t* o0, uint16_t* o1, uint16_t* o2) {
    if (dim % 4 != 0) return 4;
    for (int64_t m = 0; m < batch; ++m) {
        float bs = orc_f16_to_f32(scale_m[m]) * down_m;
        for (int64_t n = 0; n < dim; ++n) {
            float t = (float)acc[m * dim + n] * orc_f16_to_f32(scale_n[n]);
            t = t * down_n; t = t * bs;
            uint16_t h = orc_f32_to_f16(t);
            if (bias) h = orc_f16_add(h, bias[n]);
            int64_t g = n & ~(int64_t)3;                     /* split.cu:73-79: a 4-column group goes where its first column goes */
            if (g < d0) o0[m * d0 + n] = h;
            else if (g < d0 + d1) o1[m * d1 + (n - d0)] = h;
            else if (g < d0 + d1 + d2) o2[m * d2 + (n - d0 - d1)] = h;
        }
    }
    return 0;
}
