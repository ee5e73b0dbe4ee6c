// int8 x int8 -> int32 GEMM with fused dequant epilogue on the 5th-generation tensor cores
// (tcgen05.mma kind::i8, accumulators in TMEM, operands fed by TMA into 128B-swizzled shared
// memory).  Replaces the reference's cuBLASLt call (src/ppl/kernel/llm/cuda/cublas/gemm.cu:171-363)
// and the dequantize launch that follows it (src/ppl/kernel/llm/cuda/pmx/i8i8/quantize.cu:126-169).
//
// C[M,N] = A[M,K] * B[N,K]^T, both operands K-major (row-major [rows, K]), exactly the
// transa = false / transb = true convention of the reference's linear ops.
//
// Kernel shape: persistent, one CTA per SM, 6 warps:
//   warp 0      TMA producer     (one elected lane)
//   warp 1      MMA issuer       (one elected lane); also owns TMEM alloc / dealloc
//   warps 2..5  epilogue         (tcgen05.ld -> scale -> fp16 -> global), one TMEM lane quarter each
// Shared-memory ring of STAGES x {A tile 128 x 128 B, B tile BN x 128 B}; two TMEM accumulator
// buffers of BN columns each so the epilogue of tile i overlaps the main loop of tile i + 1.
// No TMA multicast is used anywhere.
#include "common.cuh"
#include "ptx.cuh"

#include <mutex>
#include <string.h>

namespace pplb200 {

namespace {

constexpr int BM = 128;       // tile rows (TMEM lanes)
constexpr int BK = 128;       // bytes (= int8 elements) of K per stage: one 128-byte swizzle row
constexpr int UMMA_K = 32;    // K per tcgen05.mma kind::i8
// warp 0: TMA producer, warp 1: MMA issuer, warps 2..: epilogue.  Four epilogue warps (one per TMEM
// lane quarter) drain a 128 x 256 accumulator faster than its successor is produced; on the
// power-capped part eight warps measured slower (more issue activity, lower clocks).
constexpr int EPI_WARPS = 4;
constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;

// status bits recorded when a bounded wait gives up
constexpr unsigned ST_PRODUCER_TIMEOUT = 1u, ST_MMA_FULL_TIMEOUT = 2u, ST_MMA_ACC_TIMEOUT = 4u, ST_EPI_TIMEOUT = 8u;

__device__ unsigned int g_gemm_status = 0;

struct KernelParams {
    int32_t M, N;
    int32_t num_m_tiles, num_n_tiles, num_k_blocks;
    int32_t mode;
    void* out; int64_t ldc;
    const half* scale_m; const half* scale_n; const half* bias;
    float down_m, down_n;
    uint32_t* row_absmax_bits;
    unsigned int* status;
    // optional diagnostics: 8 x uint64 per CTA (cycles the MMA / producer / epilogue threads spent in their waits)
    unsigned long long* stall;
    // EPI_RAW_I32 with raw_affine != 0: out = raw_alpha * acc + raw_beta * out + raw_bias[n] (wrapping int32)
    int32_t raw_affine, raw_alpha, raw_beta;
    const int32_t* raw_bias;
    // EPI_SWIGLU_F16 (CTA-pair kernel only): B = [x rows | gate rows], act_dim rows each
    int32_t act_dim;
    float beta;
    // EPI_PUSH_I32 (CTA-pair kernel only): see GemmArgs
    int32_t* push_base[kMaxPeers];
    int32_t push_rows, push_rank;
    // CTA-pair kernel, K slices of the leftover tiles (see WorkIter): tiles [0, full_tiles) are computed whole; each
    // later tile as k_slices items whose int32 partial tiles are added into sk_scratch[tile - full_tiles][256][256];
    // sk_arrivals[(tile - full_tiles) * 8 + cta * 4 + warp] counts the slices delivered.
    int32_t full_tiles, k_slices;
    // CTA-pair kernel: tiles are numbered m-tile fastest within groups of group_m m-tiles (see tile_coords)
    int32_t group_m;
    unsigned int* sk_arrivals;
    int32_t* sk_scratch;
    // EPI_GATHER_F16 (CTA-pair kernel only): see GemmArgs
    int32_t gather_ranks;
    int64_t gather_col0;
};

template <int BN> struct Cfg {
    static constexpr int A_BYTES = BM * BK;
    static constexpr int B_BYTES = BN * BK;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // the epilogue's staging buffers (EPI_STAGE_BYTES of static shared memory) come on top of the ring
    static constexpr int STAGES = (BN >= 256) ? 4 : (BN >= 128) ? 6 : 8;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024; // + slack to align the ring to 1024 B
    static constexpr int TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;
    static_assert(BN % 64 == 0 && BN >= 64 && BN <= 256, "UMMA N for M = 128; the epilogue stores 64-column slabs");
    // More than half of the SM's shared memory: at most one CTA per SM, so two CTAs can never
    // compete for (and block on) the same SM's tensor memory.
    static_assert(SMEM_BYTES > 116 * 1024 && SMEM_BYTES <= 227 * 1024, "smem budget");
};

// Dequantize + optional bias for 8 consecutive columns; returns packed halves.
template <bool ABSMAX>
__device__ __forceinline__ uint4 dequant8(const uint32_t* acc, const half* sn8, const half* bias8, float down_n,
                                          float batch_scale, bool has_bias, __half2& running_absmax) {
    uint4 ov;
    __half2* o = reinterpret_cast<__half2*>(&ov);
    const uint4 snv = *reinterpret_cast<const uint4*>(sn8);
    const __half2* sn = reinterpret_cast<const __half2*>(&snv);
    uint4 bv = make_uint4(0, 0, 0, 0);
    if (has_bias) bv = *reinterpret_cast<const uint4*>(bias8);
    const __half2* b = reinterpret_cast<const __half2*>(&bv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        // three separately rounded fp32 products in the reference's order, then fp16, then fp16 bias add
        const float2 s2 = __half22float2(sn[j]);
        float t0 = __fmul_rn((float)(int32_t)acc[2 * j], s2.x);
        float t1 = __fmul_rn((float)(int32_t)acc[2 * j + 1], s2.y);
        t0 = __fmul_rn(t0, down_n);
        t1 = __fmul_rn(t1, down_n);
        t0 = __fmul_rn(t0, batch_scale);
        t1 = __fmul_rn(t1, batch_scale);
        __half2 h = __floats2half2_rn(t0, t1);
        if (has_bias) h = __hadd2(h, b[j]);
        o[j] = h;
        if (ABSMAX) running_absmax = __hmax2(running_absmax, __habs2(h));
    }
    return ov;
}

__device__ __forceinline__ uint4 ld_shared_v4_epi(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

// Epilogue staging: every epilogue warp owns two 4 KiB buffers (32 rows x 128 bytes, 128-byte swizzle) that it
// fills from its 32 TMEM lanes and hands to the TMA unit, which writes whole 128-byte lines and clips the box
// at the matrix bounds (no per-element predicates, no partial sectors).
constexpr int EPI_STAGE_BYTES = 4 * 2 * 4096;

// accumulator columns c .. c + 31 of this lane's row: from tensor memory, or (sums != nullptr) from this lane's row
// of a K-sliced tile's summed int32 scratch (written by other SMs' reductions: loads that bypass L1)
__device__ __forceinline__ void load_sums32(const int32_t* sums, int c, int4 (&v)[8]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __ldcg(reinterpret_cast<const int4*>(sums + c) + j);
}
__device__ __forceinline__ void load_acc32(uint32_t taddr_row, const int32_t* sums, int c, uint32_t (&acc)[32]) {
    if (sums == nullptr) {
        ptx::tmem_ld_32x32(taddr_row + c, acc);
        ptx::tmem_ld_wait();
    } else {
        int4 v[8];
        load_sums32(sums, c, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            acc[4 * j] = (uint32_t)v[j].x; acc[4 * j + 1] = (uint32_t)v[j].y; acc[4 * j + 2] = (uint32_t)v[j].z; acc[4 * j + 3] = (uint32_t)v[j].w;
        }
    }
}
// the same with the scratch columns fetched one step ahead: `ahead` holds columns c .. c + 31 on entry and, when there
// is a next step, columns c + 32 .. c + 63 on return, so that their latency runs under this step's epilogue work
__device__ __forceinline__ void load_acc32_ahead(uint32_t taddr_row, const int32_t* sums, int c, bool more, int4 (&ahead)[8],
                                                 uint32_t (&acc)[32]) {
    if (sums == nullptr) {
        ptx::tmem_ld_32x32(taddr_row + c, acc);
        ptx::tmem_ld_wait();
        return;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        acc[4 * j] = (uint32_t)ahead[j].x; acc[4 * j + 1] = (uint32_t)ahead[j].y;
        acc[4 * j + 2] = (uint32_t)ahead[j].z; acc[4 * j + 3] = (uint32_t)ahead[j].w;
    }
    if (more) load_sums32(sums, c + 32, ahead);
}

// Drains this warp's 32 lanes x BN accumulator columns (TMEM address taddr_row) for output rows
// row0 .. row0 + 31 and columns n_base .. n_base + BN - 1: RAW_I32, DEQUANT_F16 or DEQUANT_F16_REQUANT_I8.
// `stage` = shared-memory address of the warp's two buffers; `sel` counts the slabs stored so far.
// `sums`: see load_acc32.
template <int BN>
__device__ __forceinline__ void drain_tile(const KernelParams& p, const CUtensorMap* tmap_out, uint32_t taddr_row,
                                           int row0, int n_base, int lane, uint32_t stage, uint32_t& sel,
                                           const int32_t* sums = nullptr) {
    const int row = row0 + lane;
    const bool row_ok = row < p.M;
    const uint32_t my_row = (uint32_t)lane * 128u, sw = (uint32_t)(lane & 7);
    int4 ahead[8];
    if (sums != nullptr) load_sums32(sums, 0, ahead);
    if (p.mode == EPI_RAW_I32) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
            const int n0 = n_base + c0;
            if (n0 >= p.N) break; // warp-uniform
            uint32_t acc[32];
            load_acc32_ahead(taddr_row, sums, c0, c0 + 32 < BN, ahead, acc);
            if (p.raw_affine) {
                const int32_t* old = reinterpret_cast<const int32_t*>(p.out) + (int64_t)row * p.ldc + n0;
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    if (n0 + j >= p.N) break; // N % 8 == 0: groups of four are all-or-nothing
                    int4 b4 = make_int4(0, 0, 0, 0), o4 = make_int4(0, 0, 0, 0);
                    if (p.raw_bias != nullptr) b4 = *reinterpret_cast<const int4*>(p.raw_bias + n0 + j);
                    if (p.raw_beta != 0 && row_ok) o4 = *reinterpret_cast<const int4*>(old + j);
                    acc[j] = (uint32_t)p.raw_alpha * acc[j] + (uint32_t)p.raw_beta * (uint32_t)o4.x + (uint32_t)b4.x;
                    acc[j + 1] = (uint32_t)p.raw_alpha * acc[j + 1] + (uint32_t)p.raw_beta * (uint32_t)o4.y + (uint32_t)b4.y;
                    acc[j + 2] = (uint32_t)p.raw_alpha * acc[j + 2] + (uint32_t)p.raw_beta * (uint32_t)o4.z + (uint32_t)b4.z;
                    acc[j + 3] = (uint32_t)p.raw_alpha * acc[j + 3] + (uint32_t)p.raw_beta * (uint32_t)o4.w + (uint32_t)b4.w;
                }
            }
            const uint32_t buf = stage + (sel & 1u) * 4096u;
            if (lane == 0) ptx::bulk_wait_group_read<1>(); // the store that last used this buffer has read it
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 8; ++j)
                ptx::st_shared_v4(buf + my_row + (((uint32_t)j ^ sw) << 4), make_uint4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]));
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && row0 < p.M) {
                ptx::tma_store_2d(tmap_out, buf, n0, row0);
                ptx::bulk_commit_group();
            }
            ++sel;
        }
        return;
    }
    const bool has_bias = p.bias != nullptr;
    const bool want_absmax = p.mode == EPI_DEQUANT_F16_REQUANT_I8;
    const float batch_scale = row_ok ? __fmul_rn(__half2float(p.scale_m[row]), p.down_m) : 0.0f;
    __half2 absmax2 = __float2half2_rn(0.0f);
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 64) {
        const int n0 = n_base + c0;
        if (n0 >= p.N) break; // warp-uniform
        const uint32_t buf = stage + (sel & 1u) * 4096u;
        if (lane == 0) ptx::bulk_wait_group_read<1>();
        __syncwarp();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int nn = n0 + 32 * h;
            if (nn >= p.N) break; // warp-uniform; the box is clipped at column N
            uint32_t acc[32];
            load_acc32_ahead(taddr_row, sums, c0 + 32 * h, c0 + 32 * h + 32 < BN, ahead, acc);
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                if (nn + j >= p.N) break;
                const uint4 v = want_absmax ? dequant8<true>(acc + j, p.scale_n + nn + j, p.bias + nn + j, p.down_n, batch_scale, has_bias, absmax2)
                                            : dequant8<false>(acc + j, p.scale_n + nn + j, p.bias + nn + j, p.down_n, batch_scale, has_bias, absmax2);
                ptx::st_shared_v4(buf + my_row + (((uint32_t)(4 * h + (j >> 3)) ^ sw) << 4), v);
            }
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && row0 < p.M) {
            ptx::tma_store_2d(tmap_out, buf, n0, row0);
            ptx::bulk_commit_group();
        }
        ++sel;
    }
    if (want_absmax && row_ok) {
        const __half m = __hmax(__low2half(absmax2), __high2half(absmax2));
        atomicMax(p.row_absmax_bits + row, __float_as_uint(__half2float(m)));
    }
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_i8_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_out, const KernelParams p) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(1024) uint8_t epi_stage[EPI_STAGE_BYTES];
    __shared__ __align__(8) uint64_t full_bar[C::STAGES];
    __shared__ __align__(8) uint64_t empty_bar[C::STAGES];
    __shared__ __align__(8) uint64_t acc_full_bar[2];
    __shared__ __align__(8) uint64_t acc_empty_bar[2];
    __shared__ uint32_t tmem_base_slot;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t ring = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;

    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
        for (int s = 0; s < C::STAGES; ++s) {
            ptx::mbar_init(ptx::smem_addr(&full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_addr(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_addr(&acc_full_bar[b]), 1);
            ptx::mbar_init(ptx::smem_addr(&acc_empty_bar[b]), EPI_WARPS);
        }
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_addr(&tmem_base_slot), C::TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    const int num_tiles = p.num_m_tiles * p.num_n_tiles;
    const int nkb = p.num_k_blocks;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m_tile = tile % p.num_m_tiles;
                const int n_tile = tile / p.num_m_tiles;
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!ptx::mbar_wait(ptx::smem_addr(&empty_bar[stage]), phase ^ 1u, p.status, ST_PRODUCER_TIMEOUT)) {
                        ok = false;
                        break;
                    }
                    const uint32_t full = ptx::smem_addr(&full_bar[stage]);
                    const uint32_t sa = ring + stage * C::STAGE_BYTES;
                    ptx::mbar_arrive_expect_tx(full, C::STAGE_BYTES);
                    ptx::tma_load_2d(sa, &tmap_a, full, kb * BK, m_tile * BM);
                    ptx::tma_load_2d(sa + C::A_BYTES, &tmap_b, full, kb * BK, n_tile * BN);
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        // One thread feeds the tensor cores, so its own instruction stream must stay well under the 128 cycles
        // an MMA takes: descriptors are a 32-bit add away from the previous ones, and the barrier of the NEXT
        // stage is polled before the current stage's MMAs are issued, so its latency hides behind them.
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::make_i8_idesc(BM, BN);
            const uint32_t a_lo0 = ptx::desc_lo_sw128(ring), full0 = ptx::smem_addr(&full_bar[0]), empty0 = ptx::smem_addr(&empty_bar[0]);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            int it = 0;
            bool ready = false;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
                const uint32_t buf = it & 1, acc_phase = (it >> 1) & 1;
                if (!ptx::mbar_wait(ptx::smem_addr(&acc_empty_bar[buf]), acc_phase ^ 1u, p.status, ST_MMA_ACC_TIMEOUT)) break;
                ptx::tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!ready && !ptx::mbar_wait(full0 + stage * 8u, phase, p.status, ST_MMA_FULL_TIMEOUT)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    uint32_t nstage = stage + 1, nphase = phase;
                    if (nstage == C::STAGES) { nstage = 0; nphase ^= 1u; }
                    ready = ptx::mbar_try_wait(full0 + nstage * 8u, nphase); // used in the next iteration
                    const uint32_t a_lo = a_lo0 + stage * (uint32_t)(C::STAGE_BYTES >> 4), b_lo = a_lo + (uint32_t)(C::A_BYTES >> 4);
                    ptx::mma_i8(tmem_d, ptx::desc_from_lo(a_lo), ptx::desc_from_lo(b_lo), idesc, kb != 0 ? 1u : 0u);
#pragma unroll
                    for (uint32_t k = 1; k < BK / UMMA_K; ++k) // +32 bytes of K = +2 in descriptor address units
                        ptx::mma_i8(tmem_d, ptx::desc_from_lo(a_lo + 2u * k), ptx::desc_from_lo(b_lo + 2u * k), idesc, 1u);
                    ptx::mma_commit(empty0 + stage * 8u); // frees the smem slot when these MMAs retire
                    stage = nstage; phase = nphase;
                }
                if (ok) ptx::mma_commit(ptx::smem_addr(&acc_full_bar[buf]));
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const int quarter = warp & 3; // TMEM lanes [32 * quarter, 32 * quarter + 32) belong to this warp
        const uint32_t stage = ptx::smem_addr(epi_stage) + (uint32_t)(warp - 2) * 8192u;
        uint32_t sel = 0;
        if (lane == 0) ptx::prefetch_tensormap(&tmap_out);
        int it = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
            const int m_tile = tile % p.num_m_tiles;
            const int n_tile = tile / p.num_m_tiles;
            const uint32_t buf = it & 1, acc_phase = (it >> 1) & 1;
            if (!ptx::mbar_wait(ptx::smem_addr(&acc_full_bar[buf]), acc_phase, p.status, ST_EPI_TIMEOUT)) break;
            ptx::tc_fence_after();
            const uint32_t taddr_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
            drain_tile<BN>(p, &tmap_out, taddr_row, m_tile * BM + quarter * 32, n_tile * BN, lane, stage, sel);

            // accumulator buffer drained: hand it back to the MMA warp
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_addr(&acc_empty_bar[buf]));
        }
        if (lane == 0) ptx::bulk_wait_group<0>(); // the staging buffers must outlive the stores that read them
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}


// Tile number -> (m tile, n tile) of the CTA-pair kernel.  Consecutive numbers run at the same time, so the numbering
// decides what is live in L2: within a group of group_m m-tiles the m index runs fastest, the n index next, and the
// groups follow one another.  With one group (all m-tiles) every wave touches the whole activation matrix, which
// for a large batch does not survive in L2 between waves next to the streaming output; with groups, the group's
// activation panels stay resident while the weight panels stream past them once per group.
__device__ __forceinline__ void tile_coords(const KernelParams& p, int tile, int& m_tile, int& n_tile) {
    const int per_group = p.group_m * p.num_n_tiles;
    const int g = tile / per_group;
    const int idx = tile - g * per_group;
    const int m0 = g * p.group_m;
    const int gm = p.num_m_tiles - m0 < p.group_m ? p.num_m_tiles - m0 : p.group_m;
    n_tile = idx / gm;
    m_tile = m0 + idx - n_tile * gm;
}

// The work of one CTA pair, in order.  The persistent grid runs in waves of one tile per pair; a tile count that is not
// a multiple of the pair count would leave most pairs idle during the last wave.  So when few tiles are left over
// (at most half as many as there are pairs), each of them is cut along K into k_slices items that different pairs
// compute at the same time, and these items come FIRST: a slice is the first item of its pair, the whole tiles
// (tile = pair + wave * pairs) follow.  A slice's int32 partial tile is added into a zeroed scratch tile by the TMA
// unit's reduction; the warp that delivers the last slice of its 32 rows reads the sums back and runs the real
// epilogue (integer sums: exact in any order; nobody waits for anybody).  Coming first, all of that -- the
// reductions, the counting, the read-back -- runs under the main loop of the pair's next tile instead of after the
// end of the kernel, and slices with the same index stay in step along K, so tiles that share an operand panel
// still fetch it from L2 together.
struct WorkIter {
    int slice, tile_next, stride, full_tiles, nkb, k_slices;
    __device__ __forceinline__ WorkIter(const KernelParams& p, int num_tiles, int pair_id, int num_pairs) {
        full_tiles = p.full_tiles; nkb = p.num_k_blocks; k_slices = p.k_slices; stride = num_pairs; tile_next = pair_id;
        slice = pair_id < (num_tiles - full_tiles) * k_slices ? pair_id : -1;
    }
    // next item: K blocks [kb0, kb0 + cnt) of `tile`
    __device__ __forceinline__ bool next(int& tile, int& kb0, int& cnt) {
        if (slice >= 0) {
            const int t = slice / k_slices, s = slice - t * k_slices;
            tile = full_tiles + t;
            kb0 = (int)((long long)nkb * s / k_slices);
            cnt = (int)((long long)nkb * (s + 1) / k_slices) - kb0;
            slice = -1;
            return true;
        }
        if (tile_next >= full_tiles) return false;
        tile = tile_next; tile_next += stride; kb0 = 0; cnt = nkb;
        return true;
    }
};

// ---- CTA-pair variant ---------------------------------------------------------------------------
// Two CTAs of a cluster compute one 256 x 256 tile with tcgen05.mma.cta_group::2: each CTA stages
// its own 128 rows of A and its own 128 rows of B (half of the tile's N), the leader issues the
// MMAs, and each CTA's tensor memory receives its 128 rows of the accumulator.  Per CTA a K block
// then costs 32 KiB of operand traffic for the same 128 tensor-core cycles x 4 that the single-CTA
// 128 x 256 tile pays 48 KiB for -- the single-CTA tile is limited by the L2 -> SM operand
// bandwidth, this one is not.  No TMA multicast: every CTA fetches its own halves.
struct PairCfg {
    static constexpr int BN = 256;
    static constexpr int HALF_N = 128;
    static constexpr int A_BYTES = BM * BK;
    static constexpr int B_BYTES = HALF_N * BK;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // per CTA
    static constexpr int STAGES = 6;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
    static constexpr int TMEM_COLS = 512;                   // two accumulator buffers of 256 columns
};

// EW = number of epilogue warps (4, or 8 for the transcendental-heavy SwiGLU epilogue, where two
// warps share a TMEM lane quarter and split the columns).
template <int EW>
__global__ void __launch_bounds__(64 + 32 * EW, 1)
gemm_i8_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                            const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_sk,
                            const KernelParams p) {
    using C = PairCfg;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[C::STAGES];   // used in the leader: both CTAs' tiles have landed
    __shared__ __align__(8) uint64_t empty_bar[C::STAGES];  // per CTA: the MMAs reading this slot retired
    __shared__ __align__(8) uint64_t acc_full_bar[2];       // per CTA: accumulator buffer complete
    __shared__ __align__(8) uint64_t acc_empty_bar[2];      // used in the leader: both CTAs drained the buffer
    __shared__ uint32_t tmem_base_slot;
    // Staging of the four-warp epilogues (two 4 KiB buffers per warp): TMA-store source of the fp16 / int32
    // outputs; in EPI_PUSH_I32 a 32 x 32 int32 block per warp, to turn "one row per lane" into 128-byte
    // contiguous row segments before the stores leave for another GPU.  Unused by the eight-warp SwiGLU form.
    __shared__ __align__(1024) uint8_t epi_stage[EW == 4 ? EPI_STAGE_BYTES : 1024];

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t ring = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t rank = ptx::cluster_ctarank();
    const bool leader = rank == 0;

    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
        for (int s = 0; s < C::STAGES; ++s) {
            ptx::mbar_init(ptx::smem_addr(&full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_addr(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_addr(&acc_full_bar[b]), 1);
            ptx::mbar_init(ptx::smem_addr(&acc_empty_bar[b]), 2 * EW); // the epilogue warps of both CTAs
        }
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_addr(&tmem_base_slot), C::TMEM_COLS);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before();
    ptx::cluster_sync_all(); // barriers of both CTAs are initialised before anyone signals them
    ptx::tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    // Launched as a programmatic dependent (fused linear), everything above ran under the tail of the preceding
    // kernel; its results (quantized activations, row scales, cleared scratch) are needed from here on.  Every
    // thread waits: all of them read such data.  A no-op in an ordinary launch.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int num_pairs = (int)(gridDim.x >> 1);
    const int pair_id = (int)(blockIdx.x >> 1);
    const int num_tiles = p.num_m_tiles * p.num_n_tiles; // tiles of 256 x 256
    const int nkb = p.num_k_blocks;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            long long t_wait = 0;
            const long long t_begin = clock64();
            const uint32_t full_local0 = ptx::smem_addr(&full_bar[0]), full_leader0 = ptx::map_to_cta(full_local0, 0);
            // Activation panels are what the following waves of the group come back to; the weight panels and the output
            // stream past them.  Marked evict-last they stay (c4 -1 %, c3 -2 %; with both operands hinted, or with the
            // weights marked evict-first, nothing or worse).
            const uint64_t pol_a = ptx::l2_policy_evict_last();
            WorkIter work(p, num_tiles, pair_id, num_pairs);
            int tile, kb0, cnt;
            while (ok && work.next(tile, kb0, cnt)) {
                int m_tile, n_tile;
                tile_coords(p, tile, m_tile, n_tile);
                const int row_a = m_tile * 256 + (int)rank * BM;
                // SwiGLU: the leader stages 128 "x" weight rows, its partner the 128 "gate" rows of the same
                // output channels, so accumulator columns [0,128) and [128,256) pair up element by element
                const int row_b = p.mode == EPI_SWIGLU_F16 ? n_tile * C::HALF_N + (int)rank * p.act_dim
                                                           : n_tile * C::BN + (int)rank * C::HALF_N;
                for (int kb = kb0; kb < kb0 + cnt; ++kb) {
                    const long long tw = p.stall ? clock64() : 0;
                    if (!ptx::mbar_wait(ptx::smem_addr(&empty_bar[stage]), phase ^ 1u, p.status, ST_PRODUCER_TIMEOUT)) {
                        ok = false;
                        break;
                    }
                    if (p.stall) t_wait += clock64() - tw;
                    const uint32_t sa = ring + stage * C::STAGE_BYTES;
                    if (leader) ptx::mbar_arrive_expect_tx(full_local0 + stage * 8u, 2 * C::STAGE_BYTES);
                    ptx::tma_load_2d_pair_hint(sa, &tmap_a, full_leader0 + stage * 8u, kb * BK, row_a, pol_a);
                    ptx::tma_load_2d_pair(sa + C::A_BYTES, &tmap_b, full_leader0 + stage * 8u, kb * BK, row_b);
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (p.stall) {
                p.stall[blockIdx.x * 8 + 3] = (unsigned long long)t_wait;
                p.stall[blockIdx.x * 8 + 4] = (unsigned long long)(clock64() - t_begin);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = ptx::make_i8_idesc(256, C::BN);
            const uint32_t a_lo0 = ptx::desc_lo_sw128(ring), full0 = ptx::smem_addr(&full_bar[0]), empty0 = ptx::smem_addr(&empty_bar[0]);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            int it = 0;
            bool ready = false;
            long long t_full = 0, t_acc = 0;
            const long long t_begin = clock64();
            WorkIter work(p, num_tiles, pair_id, num_pairs);
            int tile, kb0, cnt;
            for (; ok && work.next(tile, kb0, cnt); ++it) {
                const uint32_t buf = it & 1, acc_phase = (it >> 1) & 1;
                const long long ta = p.stall ? clock64() : 0;
                if (!ptx::mbar_wait(ptx::smem_addr(&acc_empty_bar[buf]), acc_phase ^ 1u, p.status, ST_MMA_ACC_TIMEOUT)) break;
                if (p.stall) t_acc += clock64() - ta;
                ptx::tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * C::BN;
                for (int kb = 0; kb < cnt; ++kb) {
                    if (!ready) { // the poll issued one iteration ago found the stage still empty: wait for it
                        const long long tw = p.stall ? clock64() : 0;
                        if (!ptx::mbar_wait(full0 + stage * 8u, phase, p.status, ST_MMA_FULL_TIMEOUT)) {
                            ok = false;
                            break;
                        }
                        if (p.stall) t_full += clock64() - tw;
                    }
                    ptx::tc_fence_after();
                    uint32_t nstage = stage + 1, nphase = phase;
                    if (nstage == C::STAGES) { nstage = 0; nphase ^= 1u; }
                    ready = ptx::mbar_try_wait(full0 + nstage * 8u, nphase); // used in the next iteration
                    const uint32_t a_lo = a_lo0 + stage * (uint32_t)(C::STAGE_BYTES >> 4), b_lo = a_lo + (uint32_t)(C::A_BYTES >> 4);
                    ptx::mma_i8_pair(tmem_d, ptx::desc_from_lo(a_lo), ptx::desc_from_lo(b_lo), idesc, kb != 0 ? 1u : 0u);
#pragma unroll
                    for (uint32_t k = 1; k < BK / UMMA_K; ++k)
                        ptx::mma_i8_pair(tmem_d, ptx::desc_from_lo(a_lo + 2u * k), ptx::desc_from_lo(b_lo + 2u * k), idesc, 1u);
                    // one commit frees the slot in both CTAs once these MMAs retire (a signal multicast, not a load)
                    ptx::mma_commit_pair_mcast(empty0 + stage * 8u, 3);
                    stage = nstage; phase = nphase;
                }
                if (ok) ptx::mma_commit_pair_mcast(ptx::smem_addr(&acc_full_bar[buf]), 3);
            }
            if (p.stall) {
                p.stall[blockIdx.x * 8 + 0] = (unsigned long long)(clock64() - t_begin);
                p.stall[blockIdx.x * 8 + 1] = (unsigned long long)t_full;
                p.stall[blockIdx.x * 8 + 2] = (unsigned long long)t_acc;
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
        const int quarter = warp & 3;
        constexpr int COL_GROUPS = EW / 4;
        const int col_group = (warp - 2) >> 2;
        uint32_t sel = 0;
        if (EW == 4 && lane == 0 && p.mode != EPI_PUSH_I32 && p.mode != EPI_GATHER_F16) ptx::prefetch_tensormap(&tmap_out);
        int it = 0;
        long long t_accfull = 0;
        const long long t_begin = clock64();
        WorkIter work(p, num_tiles, pair_id, num_pairs);
        int tile, kb0, cnt;
        for (; work.next(tile, kb0, cnt); ++it) {
            int m_tile, n_tile;
            tile_coords(p, tile, m_tile, n_tile);
            const uint32_t buf = it & 1, acc_phase = (it >> 1) & 1;
            const long long tw = p.stall ? clock64() : 0;
            if (!ptx::mbar_wait(ptx::smem_addr(&acc_full_bar[buf]), acc_phase, p.status, ST_EPI_TIMEOUT)) break;
            if (p.stall) t_accfull += clock64() - tw;
            ptx::tc_fence_after();

            const int row = m_tile * 256 + (int)rank * BM + quarter * 32 + lane;
            const bool row_ok = row < p.M;
            float batch_scale = 0.0f;
            if (p.mode == EPI_SWIGLU_F16 && row_ok) batch_scale = __fmul_rn(__half2float(p.scale_m[row]), p.down_m);
            const uint32_t taddr_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * C::BN;
            const int32_t* sums = nullptr; // set when the accumulators come from a K-sliced tile's scratch

            if (EW == 4 && cnt < nkb) {
                // One K slice of a leftover tile: this warp's 32 x 256 partial block is ADDED into the scratch tile, 32 x 32
                // slab by slab through the staging buffers, by the TMA unit's tiled reduction (whole 128-byte lines).
                const int t = tile - p.full_tiles;
                const int srow0 = t * 256 + (int)rank * BM + quarter * 32;
                const uint32_t stage = ptx::smem_addr(epi_stage) + (uint32_t)(warp - 2) * 8192u;
                const uint32_t my_row = (uint32_t)lane * 128u, sw = (uint32_t)(lane & 7);
#pragma unroll 1
                for (int c0 = 0; c0 < C::BN; c0 += 32) {
                    uint32_t acc[32];
                    ptx::tmem_ld_32x32(taddr_row + c0, acc);
                    ptx::tmem_ld_wait();
                    const uint32_t sbuf = stage + (sel & 1u) * 4096u;
                    if (lane == 0) ptx::bulk_wait_group_read<1>(); // the copy that last used this buffer has read it
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        ptx::st_shared_v4(sbuf + my_row + (((uint32_t)j ^ sw) << 4), make_uint4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]));
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        ptx::tma_reduce_add_2d(&tmap_sk, sbuf, c0, srow0);
                        ptx::bulk_commit_group();
                    }
                    ++sel;
                }
                // the accumulator buffer is free again
                ptx::tc_fence_before();
                __syncwarp();
                unsigned int arrived = 0;
                if (lane == 0) {
                    ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_addr(&acc_empty_bar[buf]), 0));
                    // last slice of these 32 rows to arrive?  (additions performed -> fences -> count; count -> fence -> reads)
                    ptx::bulk_wait_group<0>();     // performed, not merely read from shared memory
                    ptx::fence_proxy_async_all();  // ... by the async proxy: order them before the count
                    __threadfence();
                    arrived = atomicAdd(p.sk_arrivals + t * 8 + (int)rank * 4 + quarter, 1u);
                }
                arrived = __shfl_sync(0xffffffffu, arrived, 0);
                if (arrived != (unsigned int)p.k_slices - 1u) continue;
                // this warp delivered the last slice: the sums are complete; run the epilogue proper from them
                __threadfence();
                sums = p.sk_scratch + (int64_t)(srow0 + lane) * 256;
            }

            if (p.mode == EPI_SWIGLU_F16) {
                // out[m, n] = fp16( silu_beta(dq(x)) * dq(gate) ), operation order of the reference's
                // stand-alone kernel (swiglu.cu:92-99); row maximum of the fp32 value before rounding
                float fmax_row = 0.0f;
#pragma unroll 1
                for (int c0 = col_group * (C::HALF_N / COL_GROUPS); c0 < (col_group + 1) * (C::HALF_N / COL_GROUPS); c0 += 32) {
                    const int n0 = n_tile * C::HALF_N + c0;
                    if (n0 >= p.N) break; // warp-uniform; p.N == act_dim here
                    uint32_t ax[32], ag[32];
                    ptx::tmem_ld_32x32(taddr_row + c0, ax);
                    ptx::tmem_ld_32x32(taddr_row + C::HALF_N + c0, ag);
                    ptx::tmem_ld_wait();
                    if (!row_ok) continue;
                    half* dst = reinterpret_cast<half*>(p.out) + (int64_t)row * p.ldc + n0;
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        if (n0 + j >= p.N) break;
                        const uint4 sxv = *reinterpret_cast<const uint4*>(p.scale_n + n0 + j);
                        const uint4 sgv = *reinterpret_cast<const uint4*>(p.scale_n + p.act_dim + n0 + j);
                        const half* sx = reinterpret_cast<const half*>(&sxv);
                        const half* sg = reinterpret_cast<const half*>(&sgv);
                        uint4 ov;
                        half* o = reinterpret_cast<half*>(&ov);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float x = __fmul_rn(__fmul_rn(__fmul_rn((float)(int32_t)ax[j + e], __half2float(sx[e])), p.down_n), batch_scale);
                            const float g = __fmul_rn(__fmul_rn(__fmul_rn((float)(int32_t)ag[j + e], __half2float(sg[e])), p.down_n), batch_scale);
                            const float r = __fmul_rn(__fdiv_rn(x, __fadd_rn(1.0f, __expf(__fmul_rn(-x, p.beta)))), g);
                            o[e] = __float2half_rn(r);
                            fmax_row = fmaxf(fabsf(r), fmax_row);
                        }
                        *reinterpret_cast<uint4*>(dst + j) = ov;
                    }
                }
                if (row_ok) atomicMax(p.row_absmax_bits + row, __float_as_uint(fmax_row));
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_addr(&acc_empty_bar[buf]), 0));
                continue;
            }

            if (EW == 4 && p.mode == EPI_PUSH_I32) {
                // Raw int32 tile, each row stored into the buffer of the rank that owns it.  Lane l holds
                // row l of the warp's 32 x 32 block; after the exchange through shared memory lane l
                // stores 16 bytes of row 4 i + l / 8 (i = 0..7), so a warp-wide store covers four
                // complete 128-byte lines.
                uint4* tr = reinterpret_cast<uint4*>(epi_stage + (EW == 4 ? (warp - 2) * 8192 : 0));
                const int sub = lane >> 3, chunk = lane & 7;
                int32_t* dst_row[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int r = m_tile * 256 + (int)rank * BM + quarter * 32 + 4 * i + sub;
                    dst_row[i] = nullptr;
                    if (r < p.M) {
                        const int owner = r / p.push_rows;
                        dst_row[i] = p.push_base[owner] + ((int64_t)p.push_rank * p.push_rows + (r - owner * p.push_rows)) * p.ldc;
                    }
                }
#pragma unroll 1
                for (int c0 = 0; c0 < C::BN; c0 += 32) {
                    const int n0 = n_tile * C::BN + c0;
                    if (n0 >= p.N) break; // warp-uniform
                    uint32_t acc[32];
                    load_acc32(taddr_row, sums, c0, acc);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        tr[lane * 8 + (j ^ (lane & 7))] = make_uint4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
                    __syncwarp();
                    const int col = n0 + chunk * 4;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int r = 4 * i + sub;
                        const uint4 v = tr[r * 8 + (chunk ^ (r & 7))];
                        if (dst_row[i] != nullptr && col < p.N) *reinterpret_cast<uint4*>(dst_row[i] + col) = v;
                    }
                    __syncwarp();
                }
                if (sums != nullptr) continue; // the accumulator buffer was handed back when the slice was delivered
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_addr(&acc_empty_bar[buf]), 0));
                continue;
            }

            if (EW == 4 && p.mode == EPI_GATHER_F16) {
                // Dequantized fp16 tile, stored into the gathered [M, N_total] output of EVERY rank (this rank's own
                // area included) at this rank's column offset.  A 32-row x 64-column slab goes through shared memory
                // so that each store instruction writes four whole 128-byte lines, the pattern that crosses NVLink
                // at full rate.
                const uint32_t stage = ptx::smem_addr(epi_stage) + (uint32_t)(warp - 2) * 8192u;
                const int row0 = m_tile * 256 + (int)rank * BM + quarter * 32;
                const bool has_bias = p.bias != nullptr;
                const float bscale = row_ok ? __fmul_rn(__half2float(p.scale_m[row]), p.down_m) : 0.0f;
                const uint32_t my_row = (uint32_t)lane * 128u, sw = (uint32_t)(lane & 7);
                const int sub = lane >> 3, chunk = lane & 7;
                __half2 unused = __float2half2_rn(0.0f);
#pragma unroll 1
                for (int c0 = 0; c0 < C::BN; c0 += 64) {
                    const int n0 = n_tile * C::BN + c0;
                    if (n0 >= p.N) break; // warp-uniform
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int nn = n0 + 32 * h;
                        if (nn >= p.N) break;
                        uint32_t acc[32];
                        load_acc32(taddr_row, sums, c0 + 32 * h, acc);
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            if (nn + j >= p.N) break;
                            const uint4 v = dequant8<false>(acc + j, p.scale_n + nn + j, p.bias + nn + j, p.down_n, bscale, has_bias, unused);
                            ptx::st_shared_v4(stage + my_row + (((uint32_t)(4 * h + (j >> 3)) ^ sw) << 4), v);
                        }
                    }
                    __syncwarp();
                    const int col = n0 + chunk * 8; // eight halves = 16 bytes per lane
#pragma unroll 1
                    for (int i = 0; i < 8; ++i) {
                        const int r = 4 * i + sub;
                        if (row0 + r >= p.M || col >= p.N) continue;
                        const uint4 v = ld_shared_v4_epi(stage + (uint32_t)r * 128u + (((uint32_t)chunk ^ (uint32_t)(r & 7)) << 4));
                        const int64_t off = (int64_t)(row0 + r) * p.ldc + p.gather_col0 + col;
                        for (int d = 0; d < p.gather_ranks; ++d)
                            *reinterpret_cast<uint4*>(reinterpret_cast<half*>(p.push_base[d]) + off) = v;
                    }
                    __syncwarp();
                }
                if (sums != nullptr) continue; // the accumulator buffer was handed back when the slice was delivered
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_addr(&acc_empty_bar[buf]), 0));
                continue;
            }

            if (EW == 4)
                drain_tile<C::BN>(p, &tmap_out, taddr_row, m_tile * 256 + (int)rank * BM + quarter * 32, n_tile * C::BN, lane,
                                  ptx::smem_addr(epi_stage) + (uint32_t)(warp - 2) * 8192u, sel, sums);
            if (sums != nullptr) continue; // the accumulator buffer was handed back when the slice was delivered

            // this CTA's half of the accumulator buffer is drained: tell the leader's MMA thread
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_addr(&acc_empty_bar[buf]), 0));
        }
        if (EW == 4 && lane == 0) ptx::bulk_wait_group<0>(); // the staging buffers must outlive the stores that read them
        if (p.stall && warp == 2 && lane == 0) {
            p.stall[blockIdx.x * 8 + 5] = (unsigned long long)t_accfull;
            p.stall[blockIdx.x * 8 + 6] = (unsigned long long)(clock64() - t_begin);
        }
    }

    // Neither CTA may leave while its partner can still read its shared memory or signal its barriers.
    ptx::tc_fence_before();
    ptx::cluster_sync_all();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
    }
}

// Clears the K-slice scratch.  In the fused linear it is launched as a programmatic dependent of the quantizer: it
// depends on nothing the quantizer writes, so it runs under the quantizer's last wave -- but it only EXITS after the
// quantizer has completed (the wait below), because the GEMM, its own programmatic dependent, takes the completion of
// this grid as its licence to read the quantizer's output.
__global__ void __launch_bounds__(256) zero_fill_kernel(uint4* dst, int64_t vecs) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); // the GEMM may run its preamble meanwhile
    const int64_t i0 = (int64_t)blockIdx.x * 1024 + threadIdx.x;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (i0 + j * 256 < vecs) dst[i0 + j * 256] = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("griddepcontrol.wait;" ::: "memory"); // a no-op in an ordinary launch
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
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

// [rows, K] int8 row-major with leading dimension ld (bytes); box = {128 bytes of K, box_rows}.
bool make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int64_t ld, int box_rows) {
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

// Output matrix [M, N] with leading dimension ldc (elements of elem_bytes = 2 or 4); box = 32 rows x 128 bytes,
// 128-byte swizzle: what one epilogue warp stages per store.
bool make_output_map(CUtensorMap* map, void* base, int64_t M, int64_t N, int64_t ldc, int elem_bytes) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)(ldc * elem_bytes)};
    const cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), 32u};
    const cuuint32_t elem_strides[2] = {1, 1};
    return fn(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_INT32, 2, base, dims, strides, box,
              elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Diagnostics switch (pplb200_debug_gemm_tail_split): false = whole tiles only, whatever the tile count.
int g_slice_leftover_tiles = 1; // 0 off, 1 by the launcher's rule, 2 whenever possible

// Diagnostics switch (pplb200_debug_gemm_stall_counters): device array the CTA-pair kernel fills when non-null.
unsigned long long* g_stall_counters = nullptr;

void fill_common(KernelParams& p, const GemmArgs& a, unsigned int* status) {
    p.stall = g_stall_counters;
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
}

struct DeviceInfo {
    bool ready = false;
    int sms = 0;
    unsigned int* status = nullptr;
    cudaStream_t status_stream = nullptr; // private non-blocking stream: reading the status word waits for nobody
};
std::mutex g_dev_mutex;
DeviceInfo g_dev[64];

// One-time set-up for the current device: SM count, the device address of the status word,
// and the opt-in shared-memory sizes of the kernel instantiations.
template <int BN> bool set_smem_attr() {
    return cudaFuncSetAttribute(gemm_i8_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                Cfg<BN>::SMEM_BYTES) == cudaSuccess;
}

const DeviceInfo* device_info() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceInfo& d = g_dev[dev];
    if (!d.ready) {
        if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
        void* addr = nullptr;
        if (cudaGetSymbolAddress(&addr, g_gemm_status) != cudaSuccess) return nullptr;
        d.status = static_cast<unsigned int*>(addr);
        if (cudaStreamCreateWithFlags(&d.status_stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
        if (!set_smem_attr<256>() || !set_smem_attr<128>() || !set_smem_attr<64>()) return nullptr;
        if (cudaFuncSetAttribute(gemm_i8_tcgen05_pair_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 PairCfg::SMEM_BYTES) != cudaSuccess) return nullptr;
        if (cudaFuncSetAttribute(gemm_i8_tcgen05_pair_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 PairCfg::SMEM_BYTES) != cudaSuccess) return nullptr;
        d.ready = true;
    }
    return &d;
}

template <int BN>
int32_t launch_bn(cudaStream_t stream, const GemmArgs& a, const DeviceInfo& dev) {
    CUtensorMap ta, tb, tc;
    if (!make_operand_map(&ta, a.A, a.M, a.K, a.lda, BM)) return fail(RC_DEVICE_RUNTIME_ERROR, "tensor map (A) encode failed");
    if (!make_operand_map(&tb, a.B, a.N, a.K, a.ldb, BN)) return fail(RC_DEVICE_RUNTIME_ERROR, "tensor map (B) encode failed");
    if (!make_output_map(&tc, a.out, a.M, a.N, a.ldc, a.mode == EPI_RAW_I32 ? 4 : 2))
        return fail(RC_DEVICE_RUNTIME_ERROR, "tensor map (C) encode failed");
    KernelParams p{};
    fill_common(p, a, dev.status);
    p.num_m_tiles = (int32_t)((a.M + BM - 1) / BM);
    p.num_n_tiles = (int32_t)((a.N + BN - 1) / BN);
    const int64_t tiles = (int64_t)p.num_m_tiles * p.num_n_tiles;
    const int grid = (int)(tiles < dev.sms ? tiles : dev.sms);
    gemm_i8_tcgen05_kernel<BN><<<grid, NUM_THREADS, Cfg<BN>::SMEM_BYTES, stream>>>(ta, tb, tc, p);
    return check_launch("gemm_i8_tcgen05");
}

// 256 x 256 tiles on CTA pairs (clusters of two), persistent: one pair per two SMs.
int32_t launch_pair(cudaStream_t stream, const GemmArgs& a, const DeviceInfo& dev) {
    CUtensorMap ta, tb, tc, tsk;
    memset(&tsk, 0, sizeof(tsk)); // scratch tiles of the K slices; only touched when leftover tiles are sliced
    if (!make_operand_map(&ta, a.A, a.M, a.K, a.lda, BM)) return fail(RC_DEVICE_RUNTIME_ERROR, "tensor map (A) encode failed");
    if (!make_operand_map(&tb, a.B, a.N, a.K, a.ldb, PairCfg::HALF_N)) return fail(RC_DEVICE_RUNTIME_ERROR, "tensor map (B) encode failed");
    memset(&tc, 0, sizeof(tc)); // the SwiGLU and push epilogues store with their own instructions and never touch it
    if (a.mode != EPI_SWIGLU_F16 && a.mode != EPI_PUSH_I32 && a.mode != EPI_GATHER_F16 &&
        !make_output_map(&tc, a.out, a.M, a.N, a.ldc, a.mode == EPI_RAW_I32 ? 4 : 2))
        return fail(RC_DEVICE_RUNTIME_ERROR, "tensor map (C) encode failed");
    KernelParams p{};
    fill_common(p, a, dev.status);
    p.num_m_tiles = (int32_t)((a.M + 255) / 256);
    p.num_n_tiles = (int32_t)((a.N + PairCfg::BN - 1) / PairCfg::BN);
    p.act_dim = 0; p.beta = a.beta;
    for (int i = 0; i < kMaxPeers; ++i) p.push_base[i] = a.push_base[i];
    p.push_rows = a.push_rows; p.push_rank = a.push_rank;
    p.gather_ranks = a.gather_ranks; p.gather_col0 = a.gather_col0;
    if (a.mode == EPI_SWIGLU_F16) { // a.N = 2 * act_dim weight rows; the output has act_dim columns
        p.act_dim = (int32_t)(a.N / 2);
        p.N = p.act_dim;
        p.num_n_tiles = (int32_t)((p.act_dim + PairCfg::HALF_N - 1) / PairCfg::HALF_N);
    }
    const int64_t tiles = (int64_t)p.num_m_tiles * p.num_n_tiles;
    int64_t pairs = dev.sms / 2;
    if (tiles < pairs) pairs = tiles;
    // m-tiles per group (see tile_coords): as many activation panels (256 rows x K) as fit in about 32 MB of L2 --
    // the fewer groups, the fewer passes over the weights -- but at least 9, where a wave's footprint
    // (group_m + 74 / group_m panels) is smallest.  M8192 K8192 N28672: 16 (1.265 ms with one group of 32, 1.164 ms
    // with 16, 1.186 with 10, 1.193 with 24; DRAM reads of the one-group form were 2.09 GB for 302 MB of operands).
    {
        int64_t gm = (32ll << 20) / (256 * a.K);
        if (gm < 9) gm = 9;
        if (gm > p.num_m_tiles) gm = p.num_m_tiles;
        p.group_m = (int32_t)gm;
    }
    // Few tiles left over after the full waves: cut them along K (see WorkIter), if the caller's workspace holds the
    // scratch tiles.  Not for SwiGLU (eight epilogue warps, paired accumulator halves).
    p.full_tiles = (int32_t)tiles; p.k_slices = 1;
    const int64_t rest = tiles % pairs;
    if (rest != 0 && g_slice_leftover_tiles && a.mode != EPI_SWIGLU_F16 && rest <= kSkMaxTiles && a.sk_ws != nullptr &&
        a.sk_ws_bytes >= kSkWsBytes && (reinterpret_cast<uintptr_t>(a.sk_ws) & 255) == 0) {
        int64_t f = pairs / rest;
        if (f > 8) f = 8;
        if (f > p.num_k_blocks / 4) f = p.num_k_blocks / 4; // at least four K blocks per slice
        // Worth it when the K blocks saved -- (1 - 1/f) of a tile -- outweigh what slicing costs.  The slice's epilogue
        // (reduction, waiting for it to be performed, reading the sums back) keeps the epilogue warps busy for about
        // 28 k cycles against 5 k for a whole tile, which only a long main loop of the following tile hides; measured
        // over shapes, the cost is about 1.25 K blocks' time per leftover tile plus a fixed 13.
        if (f >= 2 && (g_slice_leftover_tiles == 2 || 4 * (f - 1) * p.num_k_blocks >= f * (52 + 5 * rest))) {
            // cleared by a kernel: a memset node between two kernels costs several times as much on the stream
            const int64_t vecs = (kSkStateBytes + rest * kSkTileBytes) / 16;
            cudaLaunchConfig_t zc = {};
            zc.gridDim = dim3((unsigned)((vecs + 1023) / 1024), 1, 1);
            zc.blockDim = dim3(256, 1, 1);
            zc.stream = stream;
            cudaLaunchAttribute za;
            za.id = cudaLaunchAttributeProgrammaticStreamSerialization;
            za.val.programmaticStreamSerializationAllowed = 1;
            zc.attrs = &za;
            zc.numAttrs = a.pdl ? 1 : 0;
            if (cudaLaunchKernelEx(&zc, zero_fill_kernel, static_cast<uint4*>(a.sk_ws), vecs) != cudaSuccess)
                return fail(RC_DEVICE_RUNTIME_ERROR, "clearing the slice scratch failed: %s", cudaGetErrorString(cudaGetLastError()));
            p.sk_arrivals = static_cast<unsigned int*>(a.sk_ws);
            p.sk_scratch = reinterpret_cast<int32_t*>(static_cast<char*>(a.sk_ws) + kSkStateBytes);
            if (!make_output_map(&tsk, p.sk_scratch, rest * 256, 256, 256, 4))
                return fail(RC_DEVICE_RUNTIME_ERROR, "tensor map (slice scratch) encode failed");
            p.full_tiles = (int32_t)(tiles - rest);
            p.k_slices = (int32_t)f;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
    const bool wide_epilogue = a.mode == EPI_SWIGLU_F16;
    cfg.blockDim = dim3(wide_epilogue ? 64 + 32 * 8 : 64 + 32 * 4, 1, 1);
    cfg.dynamicSmemBytes = PairCfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = 2;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = a.pdl ? 2 : 1;
    const cudaError_t e = wide_epilogue ? cudaLaunchKernelEx(&cfg, gemm_i8_tcgen05_pair_kernel<8>, ta, tb, tc, tsk, p)
                                        : cudaLaunchKernelEx(&cfg, gemm_i8_tcgen05_pair_kernel<4>, ta, tb, tc, tsk, p);
    if (e != cudaSuccess) return fail(RC_DEVICE_RUNTIME_ERROR, "pair GEMM launch failed: %s", cudaGetErrorString(e));
    return RC_SUCCESS;
}

} // namespace

int32_t launch_gemm(cudaStream_t stream, const GemmArgs& a) {
    if (a.M == 0 || a.N == 0) return RC_SUCCESS;
    const DeviceInfo* dev = device_info();
    if (!dev) return fail(RC_DEVICE_RUNTIME_ERROR, "device set-up failed: %s", cudaGetErrorString(cudaGetLastError()));
    if (a.M > INT32_MAX - BM || a.N > INT32_MAX - 256 || a.K > INT32_MAX - BK)
        return fail(RC_UNSUPPORTED, "GEMM extent beyond 2^31");

    if (a.mode == EPI_SWIGLU_F16 || a.mode == EPI_PUSH_I32 || a.mode == EPI_GATHER_F16)
        return launch_pair(stream, a, *dev); // the caller checked the shape

    // Up to 128 tokens the op is bound by the weight stream: dedicated small-batch kernel.
    if (a.M <= 128) return launch_gemm_decode(stream, a, dev->status, a.pdl);

    // Large problems: 256 x 256 tiles on CTA pairs, as long as every pair gets at least one tile.
    if (((a.M + 255) / 256) * ((a.N + 255) / 256) >= dev->sms / 2)
        return launch_pair(stream, a, *dev);

    // Tile width: the widest tile that still gives every SM work.
    const int64_t m_tiles = (a.M + BM - 1) / BM;
    if (m_tiles * ((a.N + 255) / 256) >= dev->sms) return launch_bn<256>(stream, a, *dev);
    if (m_tiles * ((a.N + 127) / 128) >= dev->sms) return launch_bn<128>(stream, a, *dev);
    return launch_bn<64>(stream, a, *dev);
}

void set_tail_split(int mode) { g_slice_leftover_tiles = mode; }
void set_stall_counters(void* dev_ptr) { g_stall_counters = static_cast<unsigned long long*>(dev_ptr); }
unsigned long long* stall_counters() { return g_stall_counters; }

int32_t gemm_status(int32_t reset) {
    const DeviceInfo* dev = device_info();
    if (!dev) return -1;
    // Reads the word as it is now, on a private stream: no other stream of the device is waited for.  A caller
    // that asks about particular launches synchronises the streams it launched them on first.
    unsigned int v = 0;
    if (cudaMemcpyAsync(&v, dev->status, sizeof(v), cudaMemcpyDeviceToHost, dev->status_stream) != cudaSuccess ||
        cudaStreamSynchronize(dev->status_stream) != cudaSuccess)
        return -1;
    if (reset && v != 0) {
        cudaMemsetAsync(dev->status, 0, sizeof(v), dev->status_stream);
        cudaStreamSynchronize(dev->status_stream);
    }
    return (int32_t)v;
}

} // namespace pplb200
