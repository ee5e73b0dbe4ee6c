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
#include <string.h>

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
    int32_t tile_rows;      // weight rows per tile (a multiple of 8, <= 128), chosen so that the tiles fill the SMs
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
    int32_t w_stages;            // stages of the weight ring (tile_rows * 128 bytes each)
    unsigned long long* stamps;  // optional diagnostics: 8 x uint64 per CTA, global-timer stamps of its phases
};

// Shared memory is two independent TMA rings: weight tiles come from HBM (about two microseconds away under
// load), activation tiles from L2 (re-read by every CTA, about one microsecond away), so the weight ring gets
// as many stages as fit and the activation ring only what its shorter latency needs.  With one ring of
// {weights, activations} stages the activation bytes occupied half of the memory that could hold weights in
// flight, and the weight stream ran latency-bound at two thirds of the HBM rate.
constexpr int MAX_W_STAGES = 16;

template <int BT> struct DCfg {
    static constexpr int X_BYTES = BT * BK;
    // Ring depths are multiples of the number of MMA issuers, so that every use of a slot belongs to the same issuer:
    // a thread then never polls a barrier more than one phase ahead (a parity wait cannot tell phase u from u + 2).
    static constexpr int X_STAGES = BT >= 64 ? 6 : 8;
    static constexpr int RING_BYTES = SMEM_BUDGET - 1024;
    static constexpr int X_RING_OFFSET = RING_BYTES - X_STAGES * X_BYTES; // the weight ring grows from 0 up to here
    static constexpr int SMEM_BYTES = SMEM_BUDGET;
    // Two MMA-issuing threads, each with its own accumulator tile.  With at most 128 token columns an MMA is issued
    // in 53 - 64 cycles, but the thread that issues it also waits on two barriers, polls the next two and commits
    // to two per K block: about 780 cycles per K block in all, whatever the token count and wherever the operands
    // come from (measured), which capped the weight stream at two thirds of the HBM rate.  Two threads taking
    // alternate K blocks halve that; the epilogue adds the two partial tiles while it reads them.
    static constexpr int NACC = 2;
    static constexpr int TMEM_COLS = NACC * BT < 32 ? 32 : NACC * BT;
    static_assert(TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0, "tensor-memory allocation size");
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
    static_assert(X_RING_OFFSET % 1024 == 0 && X_RING_OFFSET >= 6 * BW * BK, "room for at least six full weight tiles");
    // the rings double as the receive buffer of the reduce-scatter once the main loop is over
    static_assert(PIECES * PIECE_BYTES <= RING_BYTES, "receive buffer fits the rings");
};

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

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

// Reads N columns of each of the first `valid` accumulator tiles (BT columns apart) and returns their sum.
template <int N, int NACC, int BT>
__device__ __forceinline__ void tmem_ld_sum(uint32_t taddr, uint32_t (&acc)[N], int valid) {
    TmemLd<N>::run(taddr, acc);
    ptx::tmem_ld_wait();
#pragma unroll
    for (int a = 1; a < NACC; ++a) { // one partial tile at a time: two register arrays live, not NACC
        if (a >= valid) break; // warp-uniform: that issuer had no K block
        uint32_t part[N];
        TmemLd<N>::run(taddr + a * BT, part);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] += part[j];
    }
}

// grid = (S, weight-row tiles); cluster = (S, 1, 1): the S CTAs of a cluster share one weight-row
// tile and each takes a contiguous range of K blocks.
template <int BT>
__global__ void __launch_bounds__(DCfg<BT>::NUM_THREADS, 1)
gemm_i8_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                      const __grid_constant__ CUtensorMap tmap_y, const DecodeParams p) {
    using C = DCfg<BT>;
    constexpr int NUM_THREADS = C::NUM_THREADS;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_w[MAX_W_STAGES], empty_w[MAX_W_STAGES];
    __shared__ __align__(8) uint64_t full_x[C::X_STAGES], empty_x[C::X_STAGES];
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
    const unsigned long long t_start = p.stamps ? globaltimer_ns() : 0ull;
    const int SW = p.w_stages;
    const uint32_t w_stride = (uint32_t)p.tile_rows * BK;
    const uint32_t x_ring = ring + C::X_RING_OFFSET;

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

    if (warp == 0) { // the 45 barriers are initialised by the lanes of one warp in parallel
        if (lane == 0) {
            ptx::prefetch_tensormap(&tmap_w);
            ptx::prefetch_tensormap(&tmap_x);
            ptx::mbar_init(ptx::smem_addr(&acc_full_bar), C::NACC);
        }
        if (lane < MAX_W_STAGES) {
            ptx::mbar_init(ptx::smem_addr(&full_w[lane]), 1);
            ptx::mbar_init(ptx::smem_addr(&empty_w[lane]), 1);
        }
        if (lane < C::X_STAGES) {
            ptx::mbar_init(ptx::smem_addr(&full_x[lane]), 1);
            ptx::mbar_init(ptx::smem_addr(&empty_x[lane]), 1);
        }
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
    const unsigned long long t_setup = p.stamps ? globaltimer_ns() : 0ull;

    // per-thread output column (= weight row) and its constants; these belong to the weights, not to
    // the preceding kernel, so they are fetched now and their latency hides behind the main loop
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int grp = warp >> 2; // which slice of the token columns it handles
    const int col_begin = grp * C::GROUP_COLS, col_end = col_begin + C::GROUP_COLS;
    // A tile holds tile_rows <= 128 weight rows; the MMA still spans 128 TMEM lanes, the upper ones compute on
    // whatever the rest of the shared-memory slot holds and are never read back.
    const int n = n_tile * p.tile_rows + q * 32 + lane;
    const bool n_ok = n < p.N && q * 32 + lane < p.tile_rows;
    float sn = 0.0f;
    half bias_h = __ushort_as_half((unsigned short)0x8000u); // x + (-0.0) == x for every x: no branch for "no bias"
    if (p.mode != EPI_RAW_I32 && n_ok) {
        sn = __half2float(p.scale_n[n]);
        if (p.bias != nullptr) bias_h = p.bias[n];
    }

    bool ok = true;
    if (warp == 0 && lane == 0) {
        // ---- TMA producer of the weight ring.  The first tiles do not depend on the preceding kernel: they are
        // requested before the programmatic-dependency wait.
        const uint32_t fw0 = ptx::smem_addr(&full_w[0]), ew0 = ptx::smem_addr(&empty_w[0]);
        const int prew = nkb < SW ? nkb : SW;
        for (int i = 0; i < prew; ++i) {
            ptx::mbar_arrive_expect_tx(fw0 + i * 8u, w_stride);
            ptx::tma_load_2d(ring + i * w_stride, &tmap_w, fw0 + i * 8u, PPLB200_KB(i) * BK, n_tile * p.tile_rows);
        }
        uint32_t sw = prew == SW ? 0u : (uint32_t)prew, pw = prew == SW ? 1u : 0u;
        for (int i = prew; i < nkb; ++i) {
            if (!ptx::mbar_wait(ew0 + sw * 8u, pw ^ 1u, p.status, ST_DEC_PRODUCER)) { ok = false; break; }
            ptx::mbar_arrive_expect_tx(fw0 + sw * 8u, w_stride);
            ptx::tma_load_2d(ring + sw * w_stride, &tmap_w, fw0 + sw * 8u, PPLB200_KB(i) * BK, n_tile * p.tile_rows);
            if (++sw == (uint32_t)SW) { sw = 0; pw ^= 1u; }
        }
    } else if (warp == 3 && lane == 0) {
        // ---- TMA producer of the activation ring (a thread of its own: each barrier operation costs on the order of
        // a hundred cycles, and one thread serving both rings was as slow as the MMA issue it feeds)
        const uint32_t fx0 = ptx::smem_addr(&full_x[0]), ex0 = ptx::smem_addr(&empty_x[0]);
        pdl_wait_prior_grid(); // quantized activations are written by the preceding kernel
        uint32_t sx = 0, px = 0;
        for (int i = 0; i < nkb; ++i) {
            if (i >= C::X_STAGES && !ptx::mbar_wait(ex0 + sx * 8u, px ^ 1u, p.status, ST_DEC_PRODUCER)) { ok = false; break; }
            ptx::mbar_arrive_expect_tx(fx0 + sx * 8u, C::X_BYTES);
            ptx::tma_load_2d(x_ring + sx * C::X_BYTES, &tmap_x, fx0 + sx * 8u, PPLB200_KB(i) * BK, 0);
            if (++sx == (uint32_t)C::X_STAGES) { sx = 0; px ^= 1u; }
        }
    } else if ((warp == 1 || warp == 2) && lane == 0) {
        // ---- MMA issuers: two threads, K blocks me, me + 2, ... each, accumulator tile `me`.  Their own instruction
        // streams are kept short (descriptors are a 32-bit add away from the previous ones; the barriers of the next
        // K block are polled before this block's MMAs are issued).
        constexpr uint32_t idesc = ptx::make_i8_idesc(BW, BT);
        const int me = warp - 1;
        const uint32_t w_lo0 = ptx::desc_lo_sw128(ring), x_lo0 = ptx::desc_lo_sw128(x_ring);
        const uint32_t fw0 = ptx::smem_addr(&full_w[0]), ew0 = ptx::smem_addr(&empty_w[0]);
        const uint32_t fx0 = ptx::smem_addr(&full_x[0]), ex0 = ptx::smem_addr(&empty_x[0]);
        const uint32_t tmem_d = tmem_base + (uint32_t)me * BT;
        uint32_t sw = (uint32_t)me, pw = 0, sx = (uint32_t)me, px = 0; // both rings have at least two stages
        bool ready_w = false, ready_x = false;
        for (int i = me; i < nkb; i += C::NACC) {
            if (!ready_w && !ptx::mbar_wait(fw0 + sw * 8u, pw, p.status, ST_DEC_MMA)) { ok = false; break; }
            if (!ready_x && !ptx::mbar_wait(fx0 + sx * 8u, px, p.status, ST_DEC_MMA)) { ok = false; break; }
            ptx::tc_fence_after();
            uint32_t nsw = sw + C::NACC, npw = pw, nsx = sx + C::NACC, npx = px;
            if (nsw >= (uint32_t)SW) { nsw -= (uint32_t)SW; npw ^= 1u; }
            if (nsx >= (uint32_t)C::X_STAGES) { nsx -= (uint32_t)C::X_STAGES; npx ^= 1u; }
            ready_w = ptx::mbar_try_wait(fw0 + nsw * 8u, npw);
            ready_x = ptx::mbar_try_wait(fx0 + nsx * 8u, npx);
            const uint32_t w_lo = w_lo0 + sw * (w_stride >> 4), x_lo = x_lo0 + sx * (uint32_t)(C::X_BYTES >> 4);
            const uint32_t accumulate = i != me ? 1u : 0u;
#pragma unroll
            for (uint32_t k = 0; k < BK / UMMA_K; ++k)
                ptx::mma_i8(tmem_d, ptx::desc_from_lo(w_lo + 2u * k), ptx::desc_from_lo(x_lo + 2u * k), idesc, k != 0 ? 1u : accumulate);
            ptx::mma_commit(ew0 + sw * 8u);
            ptx::mma_commit(ex0 + sx * 8u);
            sw = nsw; pw = npw; sx = nsx; px = npx;
        }
        // both issuers report on the same barrier (two arrivals): a commit when this thread issued MMAs, else a plain arrive
        if (me < nkb) { if (ok) ptx::mma_commit(ptx::smem_addr(&acc_full_bar)); }
        else ptx::mbar_arrive(ptx::smem_addr(&acc_full_bar));
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
    const unsigned long long t_main = p.stamps ? globaltimer_ns() : 0ull;

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
                tmem_ld_sum<C::LD_COLS, C::NACC, BT>(taddr_row + c0, acc, nkb < C::NACC ? nkb : C::NACC);
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
    const unsigned long long t_exchange = p.stamps ? globaltimer_ns() : 0ull;

    // ---- epilogue over the pieces this CTA owns
    const int mode = p.mode;
    const int M = p.M;
    const float down_n = p.down_n;
    // Without a K split the CTA owns its whole [tokens x tile_rows] output tile: the values are transposed through
    // shared memory (the rings are dead by now) into a dense [token][weight row] tile and leave as ONE TMA store,
    // clipped at the matrix bounds -- instead of a 2-byte (or 4-byte) store with its own address arithmetic per
    // element (lane = weight row, registers = tokens is the wrong way round for the row-major output).
    const bool staged = S == 1 && !p.raw_affine;
    const uint32_t nl = (uint32_t)(q * 32 + lane);         // weight row inside the tile
    const bool nl_ok = nl < (uint32_t)p.tile_rows;
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
                tmem_ld_sum<C::LD_COLS, C::NACC, BT>(taddr_row + c0, acc, nkb < C::NACC ? nkb : C::NACC);
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
                    if (mode == EPI_RAW_I32 && staged) {
                        if (nl_ok) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                asm volatile("st.shared.u32 [%0], %1;" ::"r"(ring + ((uint32_t)(m0 + j) * (uint32_t)p.tile_rows + nl) * 4u), "r"(v[j]) : "memory");
                        }
                    } else if (mode == EPI_RAW_I32) {
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
                        if (staged) {
                            if (nl_ok) {
#pragma unroll
                                for (int j = 0; j < 8; ++j)
                                    asm volatile("st.shared.u16 [%0], %1;" ::"r"(ring + ((uint32_t)(m0 + j) * (uint32_t)p.tile_rows + nl) * 2u), "h"(__half_as_ushort(h[j])) : "memory");
                            }
                        } else {
                            half* dst = reinterpret_cast<half*>(p.out) + (int64_t)m0 * p.ldc + n;
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                if (n_ok && m0 + j < M) dst[(int64_t)j * p.ldc] = h[j];
                        }
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
    if (staged) ptx::fence_proxy_async_smem(); // the tile written above is read by the TMA unit
    ptx::tc_fence_before();
    __syncthreads();
    if (staged && threadIdx.x == 0) {
        ptx::tma_store_2d(&tmap_y, ring, n_tile * p.tile_rows, 0);
        ptx::bulk_commit_group();
        ptx::bulk_wait_group_read<0>(); // shared memory must outlive the store's reads; the kernel boundary publishes the writes
    }
    if (p.mode == EPI_DEQUANT_F16_REQUANT_I8) {
        for (int m = threadIdx.x; m < BT && m < p.M; m += NUM_THREADS)
            if (token_absmax[m] != 0u) atomicMax(p.row_absmax_bits + m, token_absmax[m]);
    }
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
    if (p.stamps && threadIdx.x == 0) {
        const unsigned cta = blockIdx.y * gridDim.x + blockIdx.x;
        unsigned long long* st = p.stamps + (size_t)(cta < 296u ? cta : 295u) * 8;
        st[0] = t_start; st[1] = t_setup; st[2] = t_main; st[3] = t_exchange; st[4] = globaltimer_ns();
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

// Output [M, N] (fp16 or int32, leading dimension ldc elements); box = {tile_rows weight rows, BT tokens}, dense.
bool make_out_map(CUtensorMap* map, void* base, int64_t M, int64_t N, int64_t ldc, int elem_bytes, int box_cols, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)(ldc * elem_bytes)};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    return fn(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_INT32, 2, base, dims, strides, box,
              elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
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
    int max_clusters[4][9] = {}; // [token-tile variant][cluster size]: clusters the device can hold at once
};
std::mutex g_mutex;
DecDeviceInfo g_dev[64];

template <int BT> bool set_attr(int* max_clusters) {
    if (cudaFuncSetAttribute(gemm_i8_decode_kernel<BT>, cudaFuncAttributeMaxDynamicSharedMemorySize, DCfg<BT>::SMEM_BYTES) != cudaSuccess)
        return false;
    for (int s = 2; s <= 8; ++s) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)s, 64, 1);
        cfg.blockDim = dim3(DCfg<BT>::NUM_THREADS, 1, 1);
        cfg.dynamicSmemBytes = DCfg<BT>::SMEM_BYTES;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = (unsigned)s; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_i8_decode_kernel<BT>, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
        max_clusters[s] = n;
    }
    return true;
}

const DecDeviceInfo* dec_device_info() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_mutex);
    DecDeviceInfo& d = g_dev[dev];
    if (!d.ready) {
        if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
        if (!set_attr<16>(d.max_clusters[0]) || !set_attr<32>(d.max_clusters[1]) || !set_attr<64>(d.max_clusters[2]) ||
            !set_attr<128>(d.max_clusters[3]))
            return nullptr;
        d.ready = true;
    }
    return &d;
}

template <int BT>
int32_t launch_bt(cudaStream_t stream, const GemmArgs& a, const DecDeviceInfo& dev, unsigned int* status, bool pdl) {
    CUtensorMap tw, tx;
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

    // K split: one CTA per SM is resident (the rings take the whole shared memory), so split K only as
    // far as all clusters still fit in one wave; every CTA keeps at least two K blocks
    int S = dev.sms / (int)((a.N + BW - 1) / BW);
    if (S > 8) S = 8;
    if (S > p.num_k_blocks / 2) S = p.num_k_blocks / 2;
    if (S < 1) S = 1;
    // Tile height: the smallest multiple of 8 rows with which the tiles still run as one wave -- e.g. 12288 weight
    // rows: 140 tiles of 88 rows on 148 SMs instead of 96 tiles of 128 rows on 96.  With a K split the wave holds
    // as many clusters as the device can co-schedule (fewer than SMs / S: a cluster stays inside one GPC).
    int tile_rows = BW;
    {
        const int64_t cap = S == 1 ? dev.sms : dev.max_clusters[BT == 16 ? 0 : BT == 32 ? 1 : BT == 64 ? 2 : 3][S];
        if (cap > 0 && (a.N + BW - 1) / BW <= cap) {
            int64_t r = (a.N + cap - 1) / cap;
            r = (r + 7) / 8 * 8;
            if (r < 8) r = 8;
            if (r < BW) tile_rows = (int)r;
        }
    }
    p.tile_rows = tile_rows;
    p.w_stages = DCfg<BT>::X_RING_OFFSET / (tile_rows * BK);
    if (p.w_stages > MAX_W_STAGES) p.w_stages = MAX_W_STAGES;
    p.w_stages -= p.w_stages % DCfg<BT>::NACC; // see X_STAGES
    p.stamps = stall_counters();

    const int n_tiles = (int)((a.N + tile_rows - 1) / tile_rows);
    if (!make_map(&tw, a.B, a.N, a.K, a.ldb, tile_rows)) return fail(RC_DEVICE_RUNTIME_ERROR, "tensor map (W) encode failed");
    CUtensorMap ty;
    memset(&ty, 0, sizeof(ty));
    if (S == 1 && !p.raw_affine &&
        !make_out_map(&ty, a.out, a.M, a.N, a.ldc, a.mode == EPI_RAW_I32 ? 4 : 2, tile_rows, BT))
        return fail(RC_DEVICE_RUNTIME_ERROR, "tensor map (Y) encode failed");

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
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_i8_decode_kernel<BT>, tw, tx, ty, p);
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
