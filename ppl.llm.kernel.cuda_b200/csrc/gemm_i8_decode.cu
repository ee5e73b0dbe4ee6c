// Small-batch ("decode") int8 GEMM with fused dequant epilogue for M <= 128 tokens on sm_100a.
//
// The op is bound by streaming the weight matrix from HBM once, so the kernel is organised
// around keeping every SM's TMA queue full of weight bytes:
//   * operands are swapped: 128 weight rows sit on the MMA M axis (TMEM lanes) and the tokens
//     on the MMA N axis (TMEM columns, BT = 16..128), so no tensor-core work or shared memory is
//     spent on padding tokens up to 128;
//   * one CTA per SM whose whole shared memory is one TMA ring (~200 KB in flight); when there are
//     fewer weight-row tiles than SMs, K is split over a thread-block cluster of S CTAs (one
//     weight-row tile per cluster) so that all clusters still fit in one wave;
//   * the S partial accumulators are combined inside the cluster through distributed shared
//     memory (a reduce-scatter over 8-column pieces), never through global memory, and each CTA
//     runs the dequant epilogue for the pieces it owns.  Integer addition makes the result
//     independent of the split.
//   * sixteen epilogue warps: a lone warp per scheduler issues well under one instruction per clock,
//     and the epilogue is not overlapped with anything in a one-tile-per-CTA kernel;
//   * programmatic dependent launch: weight tiles (which do not depend on the preceding
//     quantizer kernel) are requested before the kernel waits for its predecessor.
// Math and operand conventions as in gemm_i8_tcgen05.cu; reference:
// src/ppl/kernel/llm/cuda/cublas/gemm.cu:171-363, src/ppl/kernel/llm/cuda/pmx/i8i8/quantize.cu:126-169.
#include "common.cuh"
#include "ptx.cuh"

#include <mutex>

namespace pplb200 {

namespace {

constexpr int BW = 128;      // weight rows per tile (TMEM lanes)
constexpr int BK = 128;      // bytes of K per stage
constexpr int UMMA_K = 32;
constexpr int PIECE_COLS = 8; // reduce-scatter granule: 32 lanes x 8 columns x 4 B = 1 KiB
constexpr int PIECE_BYTES = 32 * PIECE_COLS * 4;
constexpr int SMEM_BUDGET = 210 * 1024; // one CTA per SM: the whole shared memory is one TMA ring

constexpr unsigned ST_DEC_PRODUCER = 16u, ST_DEC_MMA = 32u, ST_DEC_EPI = 64u;

struct DecodeParams {
    int32_t M, N;           // tokens, weight rows
    int32_t num_k_blocks;
    int32_t mode;
    void* out; int64_t ldc; // [M, ldc] int32 or fp16
    const half* scale_m; const half* scale_n; const half* bias;
    float down_m, down_n;
    uint32_t* row_absmax_bits;
    unsigned int* status;
    // EPI_RAW_I32 with raw_affine != 0: out = raw_alpha * acc + raw_beta * out + raw_bias[n] (wrapping int32)
    int32_t raw_affine, raw_alpha, raw_beta;
    const int32_t* raw_bias;
};

template <int BT> struct DCfg {
    static constexpr int W_BYTES = BW * BK;
    static constexpr int X_BYTES = BT * BK;
    static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
    static constexpr int STAGES = (SMEM_BUDGET - 1024) / STAGE_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
    static constexpr int TMEM_COLS = BT < 32 ? 32 : BT;
    // A lone warp per scheduler runs the epilogue at a fraction of an instruction per clock, so
    // the accumulator columns are spread over GROUPS sets of four warps (one warp per TMEM lane
    // quarter in each set).
    static constexpr int GROUPS = BT >= 32 ? 4 : 2;
    static constexpr int NUM_THREADS = 128 * GROUPS;
    static constexpr int GROUP_COLS = BT / GROUPS;
    static constexpr int LD_COLS = GROUP_COLS < 32 ? GROUP_COLS : 32; // columns per tcgen05.ld
    static constexpr int PIECES = 4 * (BT / PIECE_COLS);
    static_assert(LD_COLS == 8 || LD_COLS == 16 || LD_COLS == 32, "tcgen05.ld shape");
    static_assert(BT == 16 || BT == 32 || BT == 64 || BT == 128, "token tile");
    static_assert(STAGES >= 3, "pipeline depth");
    // the ring doubles as the receive buffer of the reduce-scatter: (S-1) * ceil(PIECES/S) pieces
    static_assert(PIECES * PIECE_BYTES <= STAGES * STAGE_BYTES, "receive buffer fits the ring");
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void pdl_wait_prior_grid() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Per-token maximum over the 32 lanes of a warp for NV tokens held as a[0..NV) in every lane
// (halving butterfly: NV - 1 shuffles instead of NV full warp reductions).  Returns, in every lane,
// the maximum for token (lane % NV).
template <int NV>
__device__ __forceinline__ uint32_t warp_token_max(uint32_t (&a)[NV], int lane) {
#pragma unroll
    for (int off = NV / 2; off >= 1; off >>= 1) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < off; ++i) {
            const uint32_t send = upper ? a[i] : a[i + off];
            const uint32_t keep = upper ? a[i + off] : a[i];
            const uint32_t got = __shfl_xor_sync(0xffffffffu, send, off);
            a[i] = keep > got ? keep : got;
        }
    }
    uint32_t r = a[0];
#pragma unroll
    for (int off = NV; off < 32; off <<= 1) {
        const uint32_t got = __shfl_xor_sync(0xffffffffu, r, off);
        r = r > got ? r : got;
    }
    return r;
}

template <int N> struct TmemLd;
template <> struct TmemLd<32> {
    __device__ static __forceinline__ void run(uint32_t taddr, uint32_t (&r)[32]) { ptx::tmem_ld_32x32(taddr, r); }
};
template <> struct TmemLd<8> {
    __device__ static __forceinline__ void run(uint32_t taddr, uint32_t (&r)[8]) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
            : "r"(taddr)
            : "memory");
    }
};
template <> struct TmemLd<16> {
    __device__ static __forceinline__ void run(uint32_t taddr, uint32_t (&r)[16]) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr)
            : "memory");
    }
};

// grid = (S, weight-row tiles); cluster = (S, 1, 1): the S CTAs of a cluster share one weight-row
// tile and each takes a contiguous range of K blocks.
template <int BT>
__global__ void __launch_bounds__(DCfg<BT>::NUM_THREADS, 1)
gemm_i8_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                      const DecodeParams p) {
    using C = DCfg<BT>;
    constexpr int NUM_THREADS = C::NUM_THREADS;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[C::STAGES];
    __shared__ __align__(8) uint64_t empty_bar[C::STAGES];
    __shared__ __align__(8) uint64_t acc_full_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ __align__(16) float token_scale[BT];
    __shared__ uint32_t token_absmax[BT];

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t ring = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t S = cluster_nctarank();
    const uint32_t rank = cluster_ctarank();
    const int n_tile = blockIdx.y;

    // this CTA's K blocks
    const int nkb_total = p.num_k_blocks;
    const int kb0 = (int)((int64_t)nkb_total * rank / S);
    const int kb1 = (int)((int64_t)nkb_total * (rank + 1) / S);
    const int nkb = kb1 - kb0;
    // Every cluster walks its K range from a different starting block (wrapping around), so that at
    // any instant the CTAs pull different activation tiles instead of all hitting the same L2 lines.
    // Integer accumulation makes the order irrelevant.
    const int kb_rot = nkb > 0 ? (int)(blockIdx.y % (unsigned)nkb) : 0;
#define PPLB200_KB(i) (kb0 + ((i) + kb_rot >= nkb ? (i) + kb_rot - nkb : (i) + kb_rot))

    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_w);
        ptx::prefetch_tensormap(&tmap_x);
        for (int s = 0; s < C::STAGES; ++s) {
            ptx::mbar_init(ptx::smem_addr(&full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_addr(&empty_bar[s]), 1);
        }
        ptx::mbar_init(ptx::smem_addr(&acc_full_bar), 1);
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_addr(&tmem_base_slot), C::TMEM_COLS);
        ptx::tmem_relinquish();
    }
    if (threadIdx.x < BT) token_absmax[threadIdx.x] = 0u;
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    // per-thread output column (= weight row) and its constants; these belong to the weights, not to
    // the preceding kernel, so they are fetched now and their latency hides behind the main loop
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int grp = warp >> 2; // which slice of the token columns it handles
    const int col_begin = grp * C::GROUP_COLS, col_end = col_begin + C::GROUP_COLS;
    const int n = n_tile * BW + q * 32 + lane;
    const bool n_ok = n < p.N;
    float sn = 0.0f;
    half bias_h = __ushort_as_half((unsigned short)0x8000u); // x + (-0.0) == x for every x: no branch for "no bias"
    if (p.mode != EPI_RAW_I32 && n_ok) {
        sn = __half2float(p.scale_n[n]);
        if (p.bias != nullptr) bias_h = p.bias[n];
    }

    bool ok = true;
    if (warp == 0 && lane == 0) {
        // ---- TMA producer.  Weight tiles first: they do not depend on the preceding kernel.
        const int pre = nkb < C::STAGES ? nkb : C::STAGES;
        for (int i = 0; i < pre; ++i) {
            const uint32_t full = ptx::smem_addr(&full_bar[i]);
            ptx::mbar_arrive_expect_tx(full, C::STAGE_BYTES);
            ptx::tma_load_2d(ring + i * C::STAGE_BYTES, &tmap_w, full, PPLB200_KB(i) * BK, n_tile * BW);
        }
        pdl_wait_prior_grid(); // quantized activations are written by the preceding kernel
        for (int i = 0; i < pre; ++i)
            ptx::tma_load_2d(ring + i * C::STAGE_BYTES + C::W_BYTES, &tmap_x, ptx::smem_addr(&full_bar[i]), PPLB200_KB(i) * BK, 0);
        uint32_t stage = pre == C::STAGES ? 0 : pre, phase = pre == C::STAGES ? 1 : 0;
        for (int i = pre; i < nkb; ++i) {
            if (!ptx::mbar_wait(ptx::smem_addr(&empty_bar[stage]), phase ^ 1u, p.status, ST_DEC_PRODUCER)) { ok = false; break; }
            const uint32_t full = ptx::smem_addr(&full_bar[stage]);
            const uint32_t sa = ring + stage * C::STAGE_BYTES;
            ptx::mbar_arrive_expect_tx(full, C::STAGE_BYTES);
            ptx::tma_load_2d(sa, &tmap_w, full, PPLB200_KB(i) * BK, n_tile * BW);
            ptx::tma_load_2d(sa + C::W_BYTES, &tmap_x, full, PPLB200_KB(i) * BK, 0);
            if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        constexpr uint32_t idesc = ptx::make_i8_idesc(BW, BT);
        uint32_t stage = 0, phase = 0;
        for (int i = 0; i < nkb; ++i) {
            if (!ptx::mbar_wait(ptx::smem_addr(&full_bar[stage]), phase, p.status, ST_DEC_MMA)) { ok = false; break; }
            ptx::tc_fence_after();
            const uint32_t sa = ring + stage * C::STAGE_BYTES;
            const uint64_t wdesc = ptx::make_kmajor_sw128_desc(sa);
            const uint64_t xdesc = ptx::make_kmajor_sw128_desc(sa + C::W_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
                ptx::mma_i8(tmem_base, wdesc + 2u * k, xdesc + 2u * k, idesc, (i | k) != 0 ? 1u : 0u);
            ptx::mma_commit(ptx::smem_addr(&empty_bar[stage]));
            if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) ptx::mma_commit(ptx::smem_addr(&acc_full_bar));
    }
    (void)ok;
    __syncwarp();
    pdl_wait_prior_grid(); // every thread: scale_m / row_absmax come from the preceding kernel too

    if (p.mode != EPI_RAW_I32) {
        for (int m = threadIdx.x; m < BT; m += NUM_THREADS)
            token_scale[m] = m < p.M ? __fmul_rn(__half2float(p.scale_m[m]), p.down_m) : 0.0f;
    }

    // ---- all four warps: wait for this CTA's partial accumulator
    const bool acc_ready = nkb == 0 || ptx::mbar_wait(ptx::smem_addr(&acc_full_bar), 0, p.status, ST_DEC_EPI);
    ptx::tc_fence_after();
    pdl_launch_dependents();

    const uint32_t taddr_row = tmem_base + ((uint32_t)(q * 32) << 16);
    const uint32_t recv_pieces_per_owner = (C::PIECES + S - 1) / S;
    // piece index of (column chunk c, quarter q) is 4 c + q; owner = piece % S, slot = piece / S.
    // Both are tracked incrementally (no divisions in the loops): a step of one chunk adds 4.
    const uint32_t step_div = 4u / S, step_rem = 4u % S;
    const bool have_acc = nkb > 0 && acc_ready;

    if (S > 1) {
        cluster_sync_all(); // every CTA of the cluster is done reading its ring: it may now receive
        // ---- send the pieces owned by other CTAs
        const uint32_t first_piece = (uint32_t)(col_begin / PIECE_COLS) * 4u + (uint32_t)q;
        uint32_t own = first_piece % S, slot = first_piece / S;
#pragma unroll 1
        for (int c0 = col_begin; c0 < col_end; c0 += C::LD_COLS) {
            if (c0 >= p.M) break; // columns past the last token hold zeros nobody reads
            uint32_t acc[C::LD_COLS];
            if (have_acc) {
                TmemLd<C::LD_COLS>::run(taddr_row + c0, acc);
                ptx::tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < C::LD_COLS; ++j) acc[j] = 0u;
            }
#pragma unroll
            for (int s8 = 0; s8 < C::LD_COLS / PIECE_COLS; ++s8) {
                if (own != rank) {
                    const uint32_t sender_slot = rank < own ? rank : rank - 1;
                    const uint32_t local = ring + (sender_slot * recv_pieces_per_owner + slot) * PIECE_BYTES + lane * 32;
                    const uint32_t remote = map_to_cta(local, own);
                    st_cluster_v4(remote, acc[s8 * 8 + 0], acc[s8 * 8 + 1], acc[s8 * 8 + 2], acc[s8 * 8 + 3]);
                    st_cluster_v4(remote + 16, acc[s8 * 8 + 4], acc[s8 * 8 + 5], acc[s8 * 8 + 6], acc[s8 * 8 + 7]);
                }
                own += step_rem; slot += step_div;
                if (own >= S) { own -= S; slot += 1; }
            }
        }
        cluster_sync_all(); // all partial pieces have landed
    } else {
        __syncthreads(); // token_scale visible
    }

    // ---- epilogue over the pieces this CTA owns
    const int mode = p.mode;
    const int M = p.M;
    const float down_n = p.down_n;
    {
        const uint32_t first_piece = (uint32_t)(col_begin / PIECE_COLS) * 4u + (uint32_t)q;
        uint32_t own = first_piece % S, slot = first_piece / S;
#pragma unroll 1
        for (int c0 = col_begin; c0 < col_end; c0 += C::LD_COLS) {
            if (c0 >= M) break;
            uint32_t acc[C::LD_COLS];
            uint32_t absbits[C::LD_COLS]; // |y| as float bits per token column (0 where not owned)
#pragma unroll
            for (int j = 0; j < C::LD_COLS; ++j) absbits[j] = 0u;

            if (have_acc) {
                TmemLd<C::LD_COLS>::run(taddr_row + c0, acc);
                ptx::tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < C::LD_COLS; ++j) acc[j] = 0u;
            }
#pragma unroll
            for (int s8 = 0; s8 < C::LD_COLS / PIECE_COLS; ++s8) {
                if (own == rank) {
                    uint32_t v[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = acc[s8 * 8 + j];
                    for (uint32_t r = 0; r + 1 < S; ++r) { // partials of the other S - 1 CTAs
                        const uint32_t addr = ring + (r * recv_pieces_per_owner + slot) * PIECE_BYTES + lane * 32;
                        const uint4 a = ld_shared_v4(addr), b = ld_shared_v4(addr + 16);
                        v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
                        v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
                    }
                    const int m0 = c0 + s8 * 8;
                    if (mode == EPI_RAW_I32) {
                        int32_t* dst = reinterpret_cast<int32_t*>(p.out) + (int64_t)m0 * p.ldc + n;
                        const uint32_t add = (p.raw_affine && p.raw_bias != nullptr && n_ok) ? (uint32_t)p.raw_bias[n] : 0u;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (n_ok && m0 + j < M) {
                                uint32_t r = v[j];
                                if (p.raw_affine) {
                                    r = (uint32_t)p.raw_alpha * r + add;
                                    if (p.raw_beta != 0) r += (uint32_t)p.raw_beta * (uint32_t)dst[(int64_t)j * p.ldc];
                                }
                                dst[(int64_t)j * p.ldc] = (int32_t)r;
                            }
                    } else {
                        // eight independent chains, no control flow between them
                        const float4 ts0 = *reinterpret_cast<const float4*>(&token_scale[m0]);
                        const float4 ts1 = *reinterpret_cast<const float4*>(&token_scale[m0 + 4]);
                        const float ts[8] = {ts0.x, ts0.y, ts0.z, ts0.w, ts1.x, ts1.y, ts1.z, ts1.w};
                        half h[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            float t = __fmul_rn((float)(int32_t)v[j], sn);
                            t = __fmul_rn(t, down_n);
                            t = __fmul_rn(t, ts[j]);
                            h[j] = __hadd(__float2half_rn(t), bias_h);
                        }
                        half* dst = reinterpret_cast<half*>(p.out) + (int64_t)m0 * p.ldc + n;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (n_ok && m0 + j < M) dst[(int64_t)j * p.ldc] = h[j];
                        if (mode == EPI_DEQUANT_F16_REQUANT_I8) {
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const float a = n_ok ? fabsf(__half2float(h[j])) : 0.0f;
                                absbits[s8 * 8 + j] = a == a ? __float_as_uint(a) : 0u; // NaNs are dropped, as fmax does
                            }
                        }
                    }
                }
                own += step_rem; slot += step_div;
                if (own >= S) { own -= S; slot += 1; }
            }
            if (mode == EPI_DEQUANT_F16_REQUANT_I8) {
                // per-token max |y| over this warp's 32 output columns; lane t ends up with token c0 + t
                const uint32_t tok_max = warp_token_max<C::LD_COLS>(absbits, lane);
                if (lane < C::LD_COLS && c0 + lane < M && tok_max != 0u) atomicMax(&token_absmax[c0 + lane], tok_max);
            }
        }
    }

#undef PPLB200_KB
    ptx::tc_fence_before();
    __syncthreads();
    if (p.mode == EPI_DEQUANT_F16_REQUANT_I8) {
        for (int m = threadIdx.x; m < BT && m < p.M; m += NUM_THREADS)
            if (token_absmax[m] != 0u) atomicMax(p.row_absmax_bits + m, token_absmax[m]);
    }
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---- host side ---------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

bool make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int64_t ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct DecDeviceInfo {
    bool ready = false;
    int sms = 0;
};
std::mutex g_mutex;
DecDeviceInfo g_dev[64];

template <int BT> bool set_attr() {
    return cudaFuncSetAttribute(gemm_i8_decode_kernel<BT>, cudaFuncAttributeMaxDynamicSharedMemorySize, DCfg<BT>::SMEM_BYTES) == cudaSuccess;
}

const DecDeviceInfo* dec_device_info() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_mutex);
    DecDeviceInfo& d = g_dev[dev];
    if (!d.ready) {
        if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
        if (!set_attr<16>() || !set_attr<32>() || !set_attr<64>() || !set_attr<128>()) return nullptr;
        d.ready = true;
    }
    return &d;
}

template <int BT>
int32_t launch_bt(cudaStream_t stream, const GemmArgs& a, const DecDeviceInfo& dev, unsigned int* status, bool pdl) {
    CUtensorMap tw, tx;
    if (!make_map(&tw, a.B, a.N, a.K, a.ldb, BW)) return fail(RC_DEVICE_RUNTIME_ERROR, "tensor map (W) encode failed");
    if (!make_map(&tx, a.A, a.M, a.K, a.lda, BT)) return fail(RC_DEVICE_RUNTIME_ERROR, "tensor map (X) encode failed");
    DecodeParams p;
    p.M = (int32_t)a.M; p.N = (int32_t)a.N;
    p.num_k_blocks = (int32_t)((a.K + BK - 1) / BK);
    p.mode = a.mode;
    p.out = a.out; p.ldc = a.ldc;
    p.scale_m = a.scale_m; p.scale_n = a.scale_n; p.bias = a.bias;
    p.down_m = a.down_m; p.down_n = a.down_n;
    p.row_absmax_bits = a.row_absmax_bits;
    p.status = status;
    p.raw_alpha = a.raw_alpha; p.raw_beta = a.raw_beta; p.raw_bias = a.raw_bias;
    p.raw_affine = (a.raw_alpha != 1 || a.raw_beta != 0 || a.raw_bias != nullptr) ? 1 : 0;

    const int n_tiles = (int)((a.N + BW - 1) / BW);
    // K split: one CTA per SM is resident (the ring takes the whole shared memory), so split K only as
    // far as all clusters still fit in one wave; every CTA keeps at least two K blocks
    int S = dev.sms / n_tiles;
    if (S > 8) S = 8;
    if (S > p.num_k_blocks / 2) S = p.num_k_blocks / 2;
    if (S < 1) S = 1;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)S, (unsigned)n_tiles, 1);
    cfg.blockDim = dim3(DCfg<BT>::NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = DCfg<BT>::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    int na = 0;
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = (unsigned)S;
    attrs[na].val.clusterDim.y = 1;
    attrs[na].val.clusterDim.z = 1;
    ++na;
    if (pdl) {
        attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = na;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_i8_decode_kernel<BT>, tw, tx, p);
    if (e != cudaSuccess) return fail(RC_DEVICE_RUNTIME_ERROR, "decode GEMM launch failed: %s", cudaGetErrorString(e));
    return RC_SUCCESS;
}

} // namespace

int32_t launch_gemm_decode(cudaStream_t stream, const GemmArgs& a, unsigned int* status, bool pdl) {
    const DecDeviceInfo* dev = dec_device_info();
    if (!dev) return fail(RC_DEVICE_RUNTIME_ERROR, "device set-up failed: %s", cudaGetErrorString(cudaGetLastError()));
    if (a.M <= 16) return launch_bt<16>(stream, a, *dev, status, pdl);
    if (a.M <= 32) return launch_bt<32>(stream, a, *dev, status, pdl);
    if (a.M <= 64) return launch_bt<64>(stream, a, *dev, status, pdl);
    return launch_bt<128>(stream, a, *dev, status, pdl);
}

} // namespace pplb200
