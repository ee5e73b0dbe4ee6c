// Two measurement probes that give the roofline denominators this library is reported against:
//
//  * tensor_peak: every SM issues back-to-back tcgen05.mma kind::i8 on operand tiles that stay in
//    shared memory (filled once with pseudo-random bytes; no loads, no epilogue), so the launch runs
//    at the int8 issue rate of the tensor cores at whatever clock the power limit allows.  The
//    reference has no counterpart (its GEMM is cuBLASLt); the figure is the ceiling the prefill
//    GEMMs of gemm_i8_tcgen05.cu are compared with.
//  * stream_read: one launch that pulls a byte range from global memory into shared memory with
//    bulk asynchronous copies and discards it: the fastest a single launch of that size can read,
//    fixed launch / ramp / tail cost included.  The ceiling for the small-batch GEMM's weight stream.
//
// Both kernels bound every wait and report through a status word in their result record.
#include "common.cuh"
#include "ptx.cuh"
#include "../../include/pplb200_i8i8.h"

namespace pplb200 {
namespace {

constexpr int PROBE_BK = 128;
constexpr unsigned ST_PROBE_TIMEOUT = 1u;

struct ProbeResult { // one per launch, written by CTA 0
    unsigned long long cycles; // SM cycles between first issue and completion
    unsigned long long nanos;  // globaltimer over the same span
    unsigned int status;
    unsigned int copies;       // tensor_peak with loads: 32 KiB copies CTA 0 completed while the MMAs ran
};

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t hash32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
    return x;
}

// PAIR = false: one CTA per SM, M 128 x N 256.  PAIR = true: clusters of two, cta_group::2, M 256 x N 256.
// With stream_src != nullptr a second thread keeps `LOAD_STAGES` bulk copies of 32 KiB from global memory in flight into
// spare shared memory for as long as the MMAs run (nothing consumes them): the tensor cores then read their operands
// while the copy engine fills shared memory at the rate a real GEMM main loop does.
constexpr int LOAD_STAGES = 5;
constexpr int LOAD_BYTES = 32 * 1024;

__device__ __forceinline__ void probe_bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

template <bool PAIR>
__global__ void __launch_bounds__(128, 1)
tensor_peak_kernel(int mmas, int commit_pattern, int n_cols, int rotate_acc, ProbeResult* result, const uint8_t* stream_src, long long stream_chunks) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ __align__(8) uint64_t load_bar[LOAD_STAGES];
    __shared__ __align__(8) uint64_t slot_bar; // target of the periodic commits (nobody waits on it)
    __shared__ volatile int mma_done;
    __shared__ uint32_t tmem_base_slot;
    constexpr int A_BYTES = 128 * PROBE_BK;
    constexpr int B_BYTES = (PAIR ? 128 : 256) * PROBE_BK;
    constexpr int TMEM_COLS = 256;
    const int warp = threadIdx.x >> 5;
    const uint32_t ring = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t crank = PAIR ? ptx::cluster_ctarank() : 0u;

    // operand bytes: anything but zeros (data toggling is part of the power the tensor cores draw)
    uint32_t* words = reinterpret_cast<uint32_t*>(smem_raw + (ring - ptx::smem_addr(smem_raw)));
    for (int i = threadIdx.x; i < (A_BYTES + B_BYTES) / 4; i += blockDim.x)
        words[i] = hash32(i * 2654435761u + blockIdx.x * 40503u + 12345u);
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_addr(&done_bar), 1);
        for (int i = 0; i < LOAD_STAGES; ++i) ptx::mbar_init(ptx::smem_addr(&load_bar[i]), 1);
        ptx::mbar_init(ptx::smem_addr(&slot_bar), 1);
        mma_done = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        if (PAIR) { ptx::tmem_alloc_pair(ptx::smem_addr(&tmem_base_slot), TMEM_COLS); ptx::tmem_relinquish_pair(); }
        else { ptx::tmem_alloc(ptx::smem_addr(&tmem_base_slot), TMEM_COLS); ptx::tmem_relinquish(); }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // generic-proxy writes -> visible to the tensor cores
    ptx::tc_fence_before();
    if (PAIR) ptx::cluster_sync_all(); else __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    if (threadIdx.x == 0 && crank == 0) {
        const uint32_t idesc = ptx::make_i8_idesc(PAIR ? 256 : 128, n_cols);
        const uint64_t adesc = ptx::make_kmajor_sw128_desc(ring);
        const uint64_t bdesc = ptx::make_kmajor_sw128_desc(ring + A_BYTES);
        const unsigned long long c0 = clock64(), n0 = globaltimer_ns();
        // commit_pattern: bits 0-7 = commit to a barrier after every that many MMAs (0: never), as a GEMM main
        // loop does to release an operand slot; bit 8 = a second commit to the partner CTA's barrier;
        // bit 9 = one multicast commit to both CTAs instead
        const int every = commit_pattern & 255;
        const uint32_t slot = ptx::smem_addr(&slot_bar);
        for (int i = 0; i < mmas; ++i) {
            const uint32_t k = (uint32_t)i & 3u;
            // rotate_acc: K sub-block k accumulates into its own tile (columns k * 64 ...), four independent chains
            const uint32_t d = tmem_base + (rotate_acc ? k * 64u : 0u);
            if (PAIR) ptx::mma_i8_pair(d, adesc + 2u * k, bdesc + 2u * k, idesc, i > 3 ? 1u : 0u);
            else ptx::mma_i8(d, adesc + 2u * k, bdesc + 2u * k, idesc, i > 3 ? 1u : 0u);
            if (every != 0 && (i + 1) % every == 0) {
                if (!PAIR) ptx::mma_commit(slot);
                else if (commit_pattern & 512) ptx::mma_commit_pair_mcast(slot, 3);
                else {
                    ptx::mma_commit_pair(slot);
                    if (commit_pattern & 256) ptx::mma_commit_pair(ptx::map_to_cta(slot, 1));
                }
            }
        }
        if (PAIR) ptx::mma_commit_pair(ptx::smem_addr(&done_bar)); else ptx::mma_commit(ptx::smem_addr(&done_bar));
        ptx::mbar_wait(ptx::smem_addr(&done_bar), 0, &result->status, ST_PROBE_TIMEOUT);
        const unsigned long long c1 = clock64(), n1 = globaltimer_ns();
        if (blockIdx.x == 0) {
            result->cycles = c1 - c0;
            result->nanos = n1 - n0;
        }
        mma_done = 1;
    } else if (threadIdx.x == 64 && stream_src != nullptr && stream_chunks > 0) {
        // loader: LOAD_STAGES copies in flight until the MMA thread of this CTA (of the leader: see below) is done
        const uint32_t spare = ring + 64 * 1024; // past the operand tiles
        long long c = blockIdx.x % stream_chunks;
        uint32_t parity = 0;
        for (int i = 0; i < LOAD_STAGES; ++i) {
            const uint32_t bar = ptx::smem_addr(&load_bar[i]);
            ptx::mbar_arrive_expect_tx(bar, LOAD_BYTES);
            probe_bulk_load(spare + i * LOAD_BYTES, stream_src + c * LOAD_BYTES, LOAD_BYTES, bar);
            c = (c + gridDim.x) % stream_chunks;
        }
        // both CTAs of a pair watch the leader's flag (the follower through distributed shared memory)
        const uint32_t flag = ptx::map_to_cta(ptx::smem_addr(const_cast<int*>(&mma_done)), 0);
        unsigned long long copies = 0;
        for (bool stop = false; !stop;) {
            for (int i = 0; i < LOAD_STAGES && !stop; ++i) {
                const uint32_t bar = ptx::smem_addr(&load_bar[i]);
                if (!ptx::mbar_wait(bar, parity, &result->status, ST_PROBE_TIMEOUT)) { stop = true; break; }
                ptx::mbar_arrive_expect_tx(bar, LOAD_BYTES);
                probe_bulk_load(spare + i * LOAD_BYTES, stream_src + c * LOAD_BYTES, LOAD_BYTES, bar);
                c = (c + gridDim.x) % stream_chunks;
                ++copies;
            }
            parity ^= 1u;
            int done;
            if (PAIR) asm volatile("ld.volatile.shared::cluster.s32 %0, [%1];" : "=r"(done) : "r"(flag) : "memory");
            else done = mma_done;
            if (done || copies > (1ull << 26)) stop = true;
        }
        if (blockIdx.x == 0) result->copies = (unsigned int)copies;
        for (int i = 0; i < LOAD_STAGES; ++i) // drain: no copy may be in flight when the CTA exits
            ptx::mbar_wait(ptx::smem_addr(&load_bar[i]), parity, &result->status, ST_PROBE_TIMEOUT);
    }
    ptx::tc_fence_before();
    if (PAIR) ptx::cluster_sync_all(); else __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        if (PAIR) ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS); else ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- read-only stream --------------------------------------------------------------------------
constexpr int SR_CHUNK = 32 * 1024;
constexpr int SR_STAGES = 6;

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__global__ void __launch_bounds__(32, 1)
stream_read_kernel(const uint8_t* __restrict__ src, long long chunks, ProbeResult* result) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[SR_STAGES];
    const uint32_t ring = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    if (threadIdx.x != 0) return;
    atomicMin(&result->cycles, globaltimer_ns()); // stream_read: `cycles` = earliest CTA start, `nanos` = latest CTA end (ns)
    for (int s = 0; s < SR_STAGES; ++s) ptx::mbar_init(ptx::smem_addr(&full_bar[s]), 1);
    ptx::fence_mbar_init();
    // chunk c of this CTA = blockIdx.x + c * gridDim.x; SR_STAGES copies in flight, slot reused once its copy landed
    long long issued = 0, mine = (chunks - (long long)blockIdx.x + gridDim.x - 1) / gridDim.x;
    if (mine < 0) mine = 0;
    for (; issued < mine && issued < SR_STAGES; ++issued) {
        const uint32_t bar = ptx::smem_addr(&full_bar[issued]);
        ptx::mbar_arrive_expect_tx(bar, SR_CHUNK);
        bulk_load(ring + (uint32_t)issued * SR_CHUNK, src + ((long long)blockIdx.x + issued * gridDim.x) * SR_CHUNK, SR_CHUNK, bar);
    }
    for (long long c = 0; c < mine; ++c) {
        const int slot = (int)(c % SR_STAGES);
        const uint32_t bar = ptx::smem_addr(&full_bar[slot]);
        if (!ptx::mbar_wait(bar, (uint32_t)((c / SR_STAGES) & 1), &result->status, ST_PROBE_TIMEOUT)) break;
        if (issued < mine) {
            ptx::mbar_arrive_expect_tx(bar, SR_CHUNK);
            bulk_load(ring + (uint32_t)slot * SR_CHUNK, src + ((long long)blockIdx.x + issued * gridDim.x) * SR_CHUNK, SR_CHUNK, bar);
            ++issued;
        }
    }
    atomicMax(&result->nanos, globaltimer_ns());
}

} // namespace
} // namespace pplb200

using namespace pplb200;

extern "C" {

int32_t pplb200_probe_tensor_peak(pplb200_stream_t stream_, int32_t shape, int32_t mmas_per_cta, int32_t commit_pattern, const void* stream_src,
                                  int64_t stream_bytes, void* result24) {
    cudaStream_t stream = (cudaStream_t)stream_;
    // shape: bit 0 = CTA pairs; bit 1 = four accumulators in rotation (N <= 64); bits 8.. = MMA N (0: 256)
    const int32_t cta_pairs = shape & 1, rotate_acc = (shape >> 1) & 1;
    const int32_t n_cols = (shape >> 8) ? (shape >> 8) : 256;
    if (!result24 || mmas_per_cta < 1 || mmas_per_cta > (1 << 22)) return fail(RC_INVALID_VALUE, "bad probe arguments");
    if (n_cols < 16 || n_cols > 256 || n_cols % (cta_pairs ? 32 : 16) || (rotate_acc && n_cols > 64))
        return fail(RC_INVALID_VALUE, "bad MMA N for the probe");
    if (stream_src && (!aligned16(stream_src) || stream_bytes < LOAD_BYTES)) return fail(RC_INVALID_VALUE, "bad stream source");
    const uint8_t* src = (const uint8_t*)stream_src;
    const long long chunks = stream_src ? stream_bytes / LOAD_BYTES : 0;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return fail(RC_DEVICE_RUNTIME_ERROR, "device query failed");
    ProbeResult* res = (ProbeResult*)result24;
    if (cudaMemsetAsync(res, 0, sizeof(ProbeResult), stream) != cudaSuccess) return fail(RC_DEVICE_RUNTIME_ERROR, "memset failed");
    const int smem = 226 * 1024; // operands 32 / 48 KiB, spare area for the optional loads from 64 KiB up: one CTA per SM
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(128, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cudaError_t e;
    if (cta_pairs) {
        if (cudaFuncSetAttribute(tensor_peak_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return fail(RC_DEVICE_RUNTIME_ERROR, "shared-memory opt-in failed");
        cfg.gridDim = dim3((unsigned)(sms / 2 * 2), 1, 1);
        cfg.attrs = &attr; cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, tensor_peak_kernel<true>, (int)mmas_per_cta, (int)commit_pattern, (int)n_cols, (int)rotate_acc, res, src, chunks);
    } else {
        if (cudaFuncSetAttribute(tensor_peak_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return fail(RC_DEVICE_RUNTIME_ERROR, "shared-memory opt-in failed");
        cfg.gridDim = dim3((unsigned)sms, 1, 1);
        e = cudaLaunchKernelEx(&cfg, tensor_peak_kernel<false>, (int)mmas_per_cta, (int)commit_pattern, (int)n_cols, (int)rotate_acc, res, src, chunks);
    }
    if (e != cudaSuccess) return fail(RC_DEVICE_RUNTIME_ERROR, "probe launch failed: %s", cudaGetErrorString(e));
    return RC_SUCCESS;
}

int32_t pplb200_probe_stream_read(pplb200_stream_t stream_, const void* src, int64_t bytes, void* result24) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!src || !result24 || bytes < SR_CHUNK || !aligned16(src)) return fail(RC_INVALID_VALUE, "bad probe arguments");
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return fail(RC_DEVICE_RUNTIME_ERROR, "device query failed");
    ProbeResult* res = (ProbeResult*)result24;
    if (cudaMemsetAsync(res, 0, sizeof(ProbeResult), stream) != cudaSuccess ||
        cudaMemsetAsync(&res->cycles, 0xff, sizeof(res->cycles), stream) != cudaSuccess)
        return fail(RC_DEVICE_RUNTIME_ERROR, "memset failed");
    const int smem = SR_STAGES * SR_CHUNK + 1024;
    if (cudaFuncSetAttribute(stream_read_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return fail(RC_DEVICE_RUNTIME_ERROR, "shared-memory opt-in failed");
    const long long chunks = bytes / SR_CHUNK;
    const int grid = (int)(chunks < sms ? chunks : sms);
    stream_read_kernel<<<grid, 32, smem, stream>>>((const uint8_t*)src, chunks, res);
    return check_launch("stream_read probe");
}

}
