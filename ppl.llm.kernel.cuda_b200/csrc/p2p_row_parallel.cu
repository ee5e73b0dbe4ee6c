// Row-parallel i8i8 linear whose reduction runs over peer-mapped GPU memory instead of a
// collective library: the GEMM's epilogue stores every raw int32 tile straight into the buffer of
// the rank that owns those output rows (so the transfer over NVLink runs under the main loop of the
// following tiles), the owner sums the partials exactly, applies the dequant epilogue once, and the
// other ranks fetch the finished fp16 rows.
//
//   rank r, rows [r * Ms, (r + 1) * Ms), Ms = M / size
//   buffer of every rank:  | flags 4 KiB | row-maximum slots 2 MiB | recv int32 [size][Ms][N] | staging fp16 [Ms][N] |
//
//   produce : GEMM (K shard) -> tile rows of owner o go to  peer[o].recv[r]           (remote stores)
//             signal         -> peer[*].flags["partials"][r] = epoch                  (release, system scope)
//   reduce  : wait           -> flags["partials"][*] >= epoch                         (acquire, bounded)
//             recv[0] + .. + recv[size-1] -> dequant + bias -> output rows, staging
//             signal         -> peer[*].flags["rows"][r] = epoch
//   gather  : wait; output rows of every other rank <- peer[s].staging               (remote loads)
// The sharded per-token quantizer that feeds it exchanges the row maxima through the slot area
// (described at its kernel below).
//
// Same arithmetic as the unsharded fused linear (integer sums, then the three rounded products),
// hence bit-identical to it.  Replaces, for ranks of one NVLink domain, the dequantize + fp16
// all-reduce of the reference (src/ppl/kernel/llm/cuda/pmx/i8i8/row_parallel_linear.cu:28-162).
//
// Buffer reuse needs no extra barrier: a rank's next produce follows its gather, which follows
// every peer's "rows" signal, which follows that peer's reduce (the last reader of its recv buffer);
// and a rank's next reduce (the next writer of its staging) follows every peer's next "partials"
// signal, which follows that peer's gather (the last reader of this rank's staging).
//
// Every wait is bounded; on expiry a code is ORed into the context's status word, later waits
// of that context return at once, and the result is undefined until the status is cleared.
#include "common.cuh"
#include "quant_device.cuh"
#include "../../include/pplb200_i8i8.h"

#include <new>
#include <string.h>

namespace pplb200 {
namespace {

constexpr int64_t kFlagBytes = 4096;
constexpr int kStatusWord = 64;         // uint32 indices inside the flag page
constexpr int kEpochWord = 65;          // number of produce phases enqueued so far; advanced on the device,
                                        // so a captured graph of the operation can be replayed
constexpr long long kPeerWaitCycles = 4000000000LL;
constexpr int kQuantEpochWord = 66;     // number of sharded-quantizer calls completed
constexpr int kQuantDoneWord = 67;      // CTAs of the running sharded quantizer that have finished
constexpr int kGatherEpochWord = 68;    // number of column-parallel gather operations produced so far
constexpr int kFlagRowGathered = 4;     // flag rows of the column-parallel gather: "my block is in your area",
constexpr int kFlagRowConsumed = 5;     // "I have copied the gathered output out of my area"
constexpr int64_t kQuantMaxRows = 16384;
constexpr int64_t kSlotBytes = 2 * kMaxPeers * kQuantMaxRows * 8; // [parity][source rank][row] of {epoch, max|x| bits}
constexpr unsigned ST_WAIT_PARTIALS = 1u, ST_WAIT_ROWS = 2u, ST_WAIT_ROW_MAX = 4u, ST_WAIT_GATHER = 8u, ST_WAIT_CONSUMED = 16u;

struct Ctx {
    int32_t rank = 0, size = 1, device = 0;
    uint8_t* base = nullptr;
    int64_t bytes = 0;
    uint8_t* peer[kMaxPeers] = {};
    bool opened[kMaxPeers] = {};
    bool connected = false;
    // second stream and fork / join events of the two-chunk schedule (created with the context)
    cudaStream_t side = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    // local scratch through which the GEMM's CTA pairs share tiles (GemmArgs::sk_ws), one per column chunk: the two
    // chunks' GEMMs can run at the same time; nullptr = whole tiles only
    uint8_t* sk_ws = nullptr;
};

struct Peers {
    uint8_t* base[kMaxPeers];
    int32_t rank, size;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// system-scope load that is not served from this SM's L1: the line lives in another GPU's memory
__device__ __forceinline__ uint4 ld_peer_v4(const uint4* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// flags[row][src] of every peer <- epoch.  Launched after the kernel whose stores it publishes;
// the first signal of an operation advances this rank's epoch.
// Flag rows: 2 * chunk + 0 "partial sums of column chunk `chunk` delivered", 2 * chunk + 1 "finished
// rows of that chunk are in my staging area".
__global__ void p2p_signal_kernel(Peers pr, int flag_row, int advance, int epoch_word = kEpochWord) {
    __shared__ uint32_t epoch_s;
    const int t = threadIdx.x;
    if (t == 0) {
        uint32_t* mine = reinterpret_cast<uint32_t*>(pr.base[pr.rank]) + epoch_word;
        uint32_t e = *reinterpret_cast<volatile uint32_t*>(mine);
        if (advance) *reinterpret_cast<volatile uint32_t*>(mine) = ++e;
        epoch_s = e;
    }
    __syncthreads();
    if (t < pr.size) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint32_t*>(pr.base[t]) + flag_row * kMaxPeers + pr.rank, epoch_s);
    }
}

// Block-wide: returns when every rank's flag of row `flag_row` has reached this rank's epoch, or when the cycle
// budget is spent (status |= code), or at once when the status word is already set.
__device__ __forceinline__ void wait_flags(uint32_t* flag_page, int flag_row, int size, unsigned code,
                                           int epoch_word = kEpochWord) {
    if ((int)threadIdx.x < size) {
        uint32_t* status = flag_page + kStatusWord;
        const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(flag_page + epoch_word);
        const uint32_t* f = flag_page + flag_row * kMaxPeers + threadIdx.x;
        if (*reinterpret_cast<volatile uint32_t*>(status) == 0) {
            const long long t0 = clock64();
            for (uint32_t spin = 1; (int32_t)(ld_acquire_sys(f) - epoch) < 0; ++spin) {
                if ((spin & 0xffu) == 0) {
                    if (clock64() - t0 > kPeerWaitCycles) { atomicOr(status, code); break; }
                    if (*reinterpret_cast<volatile uint32_t*>(status) != 0) break;
                }
            }
        }
    }
    __syncthreads();
}

// Sums the `size` partial slices of this rank's rows over the columns [col0, col0 + ncols) and applies
// the dequant epilogue: 8 columns per item.  Writes the rows into the caller's output and into the
// staging copy (both with leading dimension `dim`).
__global__ void __launch_bounds__(256)
p2p_reduce_dequant_kernel(uint32_t* flag_page, int flag_row, int size, const int32_t* recv,
                          int64_t rows, int64_t dim, int64_t col0, int64_t ncols, const half* __restrict__ scale_m,
                          const half* __restrict__ scale_n, const half* __restrict__ bias, float down_m, float down_n,
                          half* __restrict__ out_rows, half* __restrict__ staging) {
    wait_flags(flag_page, flag_row, size, ST_WAIT_PARTIALS);
    const int64_t chunks_per_row = ncols >> 3;
    const int64_t total = rows * chunks_per_row;
    const int64_t slice = rows * dim;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / chunks_per_row;
        const int64_t n = col0 + ((i - m * chunks_per_row) << 3);
        const int32_t* src = recv + m * dim + n;
        // recv is written by other GPUs while this kernel is resident (it only reads after the acquire
        // above): relaxed system-scope loads, never the read-only path
        uint4 a0 = ld_peer_v4(reinterpret_cast<const uint4*>(src));
        uint4 a1 = ld_peer_v4(reinterpret_cast<const uint4*>(src + 4));
        for (int s = 1; s < size; ++s) {
            const uint4 b0 = ld_peer_v4(reinterpret_cast<const uint4*>(src + s * slice));
            const uint4 b1 = ld_peer_v4(reinterpret_cast<const uint4*>(src + s * slice + 4));
            a0.x += b0.x; a0.y += b0.y; a0.z += b0.z; a0.w += b0.w;
            a1.x += b1.x; a1.y += b1.y; a1.z += b1.z; a1.w += b1.w;
        }
        const float bs = __fmul_rn(__half2float(scale_m[m]), down_m);
        const uint4 snv = *reinterpret_cast<const uint4*>(scale_n + n);
        const half* sn = reinterpret_cast<const half*>(&snv);
        const int32_t a[8] = {(int32_t)a0.x, (int32_t)a0.y, (int32_t)a0.z, (int32_t)a0.w,
                              (int32_t)a1.x, (int32_t)a1.y, (int32_t)a1.z, (int32_t)a1.w};
        uint4 ov;
        half* o = reinterpret_cast<half*>(&ov);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            // three separately rounded products in the order of the fused GEMM epilogue
            float t = __fmul_rn((float)a[j], __half2float(sn[j]));
            t = __fmul_rn(t, down_n);
            t = __fmul_rn(t, bs);
            o[j] = __float2half_rn(t);
        }
        if (bias != nullptr) {
            const uint4 bv = *reinterpret_cast<const uint4*>(bias + n);
            const half* b = reinterpret_cast<const half*>(&bv);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = __hadd(o[j], b[j]);
        }
        *reinterpret_cast<uint4*>(out_rows + m * dim + n) = ov;
        *reinterpret_cast<uint4*>(staging + m * dim + n) = ov;
    }
}

// Copies the finished fp16 rows (columns [col0, col0 + ncols)) of every other rank from its staging
// area into this rank's output.  A work item is 16 bytes; consecutive groups of 256 items read
// different peers, starting with rank + 1, so all links carry traffic at once and no two ranks
// start on the same peer.  Four items per thread are in flight.
__global__ void __launch_bounds__(256)
p2p_gather_kernel(Peers pr, int flag_row, int64_t staging_offset, int64_t rows, int64_t dim, int64_t col0, int64_t ncols,
                  half* __restrict__ out) {
    wait_flags(reinterpret_cast<uint32_t*>(pr.base[pr.rank]), flag_row, pr.size, ST_WAIT_ROWS);
    const int others = pr.size - 1;
    const int64_t vec_per_row = ncols >> 3;
    const int64_t vec_per_slice = rows * vec_per_row;
    const int64_t pieces = ((vec_per_slice + 255) >> 8) * others;
    for (int64_t piece0 = blockIdx.x; piece0 < pieces; piece0 += 4 * (int64_t)gridDim.x) {
        uint4 val[4];
        uint4* dst[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int64_t piece = piece0 + u * (int64_t)gridDim.x;
            dst[u] = nullptr;
            if (piece >= pieces) continue;
            const int q = (int)(piece % others);
            const int64_t v = (piece / others) * 256 + threadIdx.x;
            if (v >= vec_per_slice) continue;
            int src = pr.rank + 1 + q;
            if (src >= pr.size) src -= pr.size;
            const int64_t m = v / vec_per_row;
            const int64_t off = m * dim + col0 + ((v - m * vec_per_row) << 3); // in halves, inside a rank's slice
            val[u] = ld_peer_v4(reinterpret_cast<const uint4*>(reinterpret_cast<const half*>(pr.base[src] + staging_offset) + off));
            dst[u] = reinterpret_cast<uint4*>(out + (int64_t)src * rows * dim + off);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (dst[u] != nullptr) *dst[u] = val[u];
    }
}

// ---- column-parallel gather ------------------------------------------------------------------
// Before a rank may store its next block into the peers' areas, every peer must have copied the previous
// gathered output out of its area: one warp waits (bounded) for their "consumed" flags of the previous operation.
__global__ void p2p_wait_consumed_kernel(uint32_t* flag_page, int size) {
    wait_flags(flag_page, kFlagRowConsumed, size, ST_WAIT_CONSUMED, kGatherEpochWord);
}

// Waits for every rank's "block delivered" flag of the current operation, then copies the gathered fp16 matrix
// (elems halves, a multiple of 8) from this rank's area into the caller's output.
__global__ void __launch_bounds__(256)
p2p_gather_copy_kernel(uint32_t* flag_page, int size, const uint4* area, int64_t vecs, uint4* __restrict__ out) {
    wait_flags(flag_page, kFlagRowGathered, size, ST_WAIT_GATHER, kGatherEpochWord);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < vecs; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = ld_peer_v4(area + i); // written by other GPUs while this kernel was resident: never the read-only path
}

// ---- sharded per-token quantizer ------------------------------------------------------------
// Every rank holds the K shard [batch, dim] of the activation rows; the row scale must come from the
// maximum over the whole row.  One persistent kernel, all CTAs resident, CTA c owns rows c, c + grid, ...
//   pass 1: shard maximum of each of its rows, published to every rank as one 8-byte word
//           {epoch, float bits} (a single store, so no ordering is needed);
//   pass 2: per row, poll the own slots until every rank's word of this epoch has arrived (by then
//           it usually has), re-read the row (from L2 for any realistic shard) and round it with the
//           global maximum -- the same arithmetic as the unsharded quantizer, hence the same int8
//           values and scales.
// A CTA publishes all its rows before it waits for any, and every CTA of the grid is resident, so
// the ranks cannot block one another.  Slots alternate between two banks by epoch parity: a rank can
// only reach epoch e + 2 after every peer finished epoch e + 1, i.e. after it read all words of epoch e.
// (A one-pass form that kept the row in registers across the exchange stalled a CTA for the full
// exchange latency on every row: 29 us for 2048 x 3584 on 8 GPUs.)
using namespace qdev;

__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

template <int UNITS>
__global__ void __launch_bounds__(QTPB)
p2p_quantize_rows_kernel(const half* __restrict__ in, int64_t batch, int64_t dim, float up_scale,
                         int8_t* __restrict__ q, half* __restrict__ scale_out, Peers pr, int publish_only) {
    __shared__ float red[QTPB / 32];
    __shared__ uint32_t epoch_s;
    __shared__ float row_max_s;
    uint32_t* flag_page = reinterpret_cast<uint32_t*>(pr.base[pr.rank]);
    uint32_t* status = flag_page + kStatusWord;
    if (threadIdx.x == 0) epoch_s = *reinterpret_cast<volatile uint32_t*>(flag_page + kQuantEpochWord) + 1u;
    __syncthreads();
    const uint32_t epoch = epoch_s;
    const int64_t bank = (int64_t)(epoch & 1u) * kMaxPeers * kQuantMaxRows;
    const int units = (int)(dim >> 4);

    uint4 v[UNITS][2];
    auto load_row = [&](int64_t row) {
        const uint4* src = reinterpret_cast<const uint4*>(in + row * dim);
#pragma unroll
        for (int u = 0; u < UNITS; ++u) {
            const int unit = u * blockDim.x + threadIdx.x;
            if (unit < units) {
                v[u][0] = src[2 * unit]; // cached: pass 2 reads the row again
                v[u][1] = src[2 * unit + 1];
            } else {
                v[u][0] = make_uint4(0, 0, 0, 0);
                v[u][1] = make_uint4(0, 0, 0, 0);
            }
        }
    };

    // ---- pass 1: shard maxima, published to every rank
    for (int64_t row = blockIdx.x; row < batch; row += gridDim.x) {
        load_row(row);
        __half2 m2 = __float2half2_rn(0.0f);
#pragma unroll
        for (int u = 0; u < UNITS; ++u) {
            const __half2* h = reinterpret_cast<const __half2*>(&v[u][0]);
#pragma unroll
            for (int i = 0; i < 8; ++i) m2 = __hmax2(m2, __habs2(h[i]));
        }
        const float shard_max = block_max(fmaxf(__low2float(m2), __high2float(m2)), red, blockDim.x >> 5);
        if ((int)threadIdx.x < pr.size) {
            unsigned long long* theirs = reinterpret_cast<unsigned long long*>(pr.base[threadIdx.x] + kFlagBytes) + bank +
                                         (int64_t)pr.rank * kQuantMaxRows + row;
            st_relaxed_sys_u64(theirs, ((unsigned long long)epoch << 32) | __float_as_uint(shard_max));
        }
        __syncthreads(); // red[] is reused by the next row
    }
    if (publish_only) return;

    // ---- pass 2: global maxima, rounding
    for (int64_t row = blockIdx.x; row < batch; row += gridDim.x) {
        load_row(row); // requested before the wait below
        if (threadIdx.x < 32) {
            float other = 0.0f;
            if ((int)threadIdx.x < pr.size) {
                const unsigned long long* mine = reinterpret_cast<const unsigned long long*>(pr.base[pr.rank] + kFlagBytes) + bank +
                                                 (int64_t)threadIdx.x * kQuantMaxRows + row;
                unsigned long long w = ld_relaxed_sys_u64(mine);
                if ((uint32_t)(w >> 32) != epoch && *reinterpret_cast<volatile uint32_t*>(status) == 0) {
                    const long long t0 = clock64();
                    for (uint32_t spin = 1;; ++spin) {
                        w = ld_relaxed_sys_u64(mine);
                        if ((uint32_t)(w >> 32) == epoch) break;
                        if ((spin & 0xffu) == 0) {
                            if (clock64() - t0 > kPeerWaitCycles) { atomicOr(status, ST_WAIT_ROW_MAX); break; }
                            if (*reinterpret_cast<volatile uint32_t*>(status) != 0) break;
                        }
                    }
                }
                other = __uint_as_float((uint32_t)w);
            }
#pragma unroll
            for (int m = 4; m >= 1; m >>= 1) other = fmaxf(other, __shfl_xor_sync(0xffffffffu, other, m));
            if (threadIdx.x == 0) row_max_s = other;
        }
        __syncthreads();
        const QuantRow qr = make_quant_row(row_max_s, false);
        const float scale = qr.scale;
#pragma unroll
        for (int u = 0; u < UNITS; ++u) {
            const int unit = u * blockDim.x + threadIdx.x;
            if (unit < units)
                *reinterpret_cast<uint4*>(q + row * dim + ((int64_t)unit << 4)) =
                    quant16<true>(reinterpret_cast<const __half2*>(&v[u][0]), qr);
        }
        if (threadIdx.x == 0) scale_out[row] = __float2half_rn(scale * up_scale);
        __syncthreads(); // row_max_s is reused by the next row
    }

    // the last CTA to finish closes the epoch
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(flag_page + kQuantDoneWord, 1u) == gridDim.x - 1) {
            flag_page[kQuantDoneWord] = 0u;
            *reinterpret_cast<volatile uint32_t*>(flag_page + kQuantEpochWord) = epoch;
        }
    }
}

int64_t recv_bytes(int64_t M, int64_t N) { return round_up(M * N * 4, 256); }
int64_t staging_bytes(int64_t M, int64_t N, int32_t size) { return round_up(M / size * N * 2, 256); }

Peers peers_of(const Ctx& c) {
    Peers p;
    for (int i = 0; i < kMaxPeers; ++i) p.base[i] = c.peer[i];
    p.rank = c.rank; p.size = c.size;
    return p;
}

} // namespace
} // namespace pplb200

using namespace pplb200;

extern "C" {

int64_t pplb200_i8i8_row_parallel_p2p_bytes(int64_t M, int64_t N, int32_t size) {
    if (M < 0 || N < 0 || size < 1 || size > kMaxPeers) return -1;
    return kFlagBytes + kSlotBytes + recv_bytes(M, N) + staging_bytes(M, N, size);
}

int32_t pplb200_p2p_create(int32_t rank, int32_t size, int64_t bytes, void** ctx_out) {
    clear_error();
    if (!ctx_out) return fail(RC_INVALID_VALUE, "ctx_out is null");
    if (size < 1 || size > kMaxPeers || rank < 0 || rank >= size) return fail(RC_INVALID_VALUE, "bad rank/size %d/%d", rank, size);
    if (bytes < kFlagBytes + kSlotBytes) return fail(RC_INVALID_VALUE, "buffer smaller than the flag and slot pages");
    Ctx* c = new (std::nothrow) Ctx;
    if (!c) return fail(RC_DEVICE_RUNTIME_ERROR, "out of host memory");
    c->rank = rank; c->size = size; c->bytes = bytes;
    if (cudaGetDevice(&c->device) != cudaSuccess || cudaMalloc((void**)&c->base, (size_t)bytes) != cudaSuccess) {
        const int32_t rc = fail(RC_DEVICE_RUNTIME_ERROR, "cudaMalloc of %lld bytes failed: %s", (long long)bytes, cudaGetErrorString(cudaGetLastError()));
        delete c;
        return rc;
    }
    if (cudaMemset(c->base, 0, (size_t)(kFlagBytes + kSlotBytes)) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        cudaFree(c->base);
        delete c;
        return fail(RC_DEVICE_RUNTIME_ERROR, "clearing the flag and slot pages failed");
    }
    if (cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->join, cudaEventDisableTiming) != cudaSuccess) {
        cudaFree(c->base);
        delete c;
        return fail(RC_DEVICE_RUNTIME_ERROR, "stream / event creation failed");
    }
    if (cudaMalloc((void**)&c->sk_ws, (size_t)(2 * kSkWsBytes)) != cudaSuccess) {
        c->sk_ws = nullptr; // optional
        cudaGetLastError();
    }
    c->peer[rank] = c->base;
    c->connected = size == 1;
    *ctx_out = c;
    return RC_SUCCESS;
}

int32_t pplb200_p2p_export(void* ctx, void* handle64_host) {
    clear_error();
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    Ctx* c = (Ctx*)ctx;
    if (!c || !handle64_host) return fail(RC_INVALID_VALUE, "null argument");
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, c->base) != cudaSuccess)
        return fail(RC_DEVICE_RUNTIME_ERROR, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(cudaGetLastError()));
    memcpy(handle64_host, &h, 64);
    return RC_SUCCESS;
}

int32_t pplb200_p2p_connect(void* ctx, const void* handles_host) {
    clear_error();
    Ctx* c = (Ctx*)ctx;
    if (!c || !handles_host) return fail(RC_INVALID_VALUE, "null argument");
    for (int r = 0; r < c->size; ++r) {
        if (r == c->rank || c->peer[r] != nullptr) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char*)handles_host + 64 * r, 64);
        void* p = nullptr;
        if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess)
            return fail(RC_DEVICE_RUNTIME_ERROR, "cudaIpcOpenMemHandle(rank %d) failed: %s", r, cudaGetErrorString(cudaGetLastError()));
        c->peer[r] = (uint8_t*)p;
        c->opened[r] = true;
    }
    c->connected = true;
    return RC_SUCCESS;
}

int32_t pplb200_p2p_connect_local(void* ctx, void* const* peer_ctx) {
    clear_error();
    Ctx* c = (Ctx*)ctx;
    if (!c || !peer_ctx) return fail(RC_INVALID_VALUE, "null argument");
    for (int r = 0; r < c->size; ++r) {
        if (r == c->rank) continue;
        const Ctx* o = (const Ctx*)peer_ctx[r];
        if (!o || o->rank != r || o->size != c->size || o->bytes != c->bytes)
            return fail(RC_INVALID_VALUE, "peer context %d does not match", r);
        if (o->device != c->device) {
            int can = 0;
            if (cudaDeviceCanAccessPeer(&can, c->device, o->device) != cudaSuccess || !can)
                return fail(RC_UNSUPPORTED, "device %d cannot access device %d", c->device, o->device);
            const cudaError_t e = cudaDeviceEnablePeerAccess(o->device, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
                return fail(RC_DEVICE_RUNTIME_ERROR, "cudaDeviceEnablePeerAccess failed: %s", cudaGetErrorString(e));
            cudaGetLastError();
        }
        c->peer[r] = o->base;
    }
    c->connected = true;
    return RC_SUCCESS;
}

int32_t pplb200_p2p_destroy(void* ctx) {
    Ctx* c = (Ctx*)ctx;
    if (!c) return RC_SUCCESS;
    cudaDeviceSynchronize();
    for (int r = 0; r < c->size; ++r)
        if (c->opened[r]) cudaIpcCloseMemHandle(c->peer[r]);
    cudaFree(c->base);
    if (c->sk_ws) cudaFree(c->sk_ws);
    if (c->side) cudaStreamDestroy(c->side);
    if (c->fork) cudaEventDestroy(c->fork);
    if (c->join) cudaEventDestroy(c->join);
    delete c;
    return RC_SUCCESS;
}

int32_t pplb200_p2p_status(void* ctx, int32_t reset) {
    Ctx* c = (Ctx*)ctx;
    if (!c) return -1;
    // read on the context's own (non-blocking) stream: no other stream of the device is waited for
    uint32_t v = 0;
    uint32_t* word = reinterpret_cast<uint32_t*>(c->base) + kStatusWord;
    if (cudaMemcpyAsync(&v, word, 4, cudaMemcpyDeviceToHost, c->side) != cudaSuccess ||
        cudaStreamSynchronize(c->side) != cudaSuccess)
        return -1;
    if (reset && v != 0) {
        cudaMemsetAsync(word, 0, 4, c->side);
        cudaStreamSynchronize(c->side);
    }
    return (int32_t)v;
}

int32_t pplb200_i8i8_row_parallel_linear_p2p(pplb200_stream_t stream_, void* ctx, const void* input, int64_t M,
                                             int64_t input_ld, const void* weight, const void* optional_bias,
                                             const void* scale_M, const void* scale_N, float down_scale_M,
                                             float down_scale_N, int64_t in_features, int64_t out_features,
                                             int32_t phases, void* output) {
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    Ctx* c = (Ctx*)ctx;
    if (!c) return fail(RC_INVALID_VALUE, "null context");
    if (!c->connected) return fail(RC_INVALID_VALUE, "context is not connected to its peers");
    const int32_t schedule = phases & 24; // 8: force the two-chunk schedule, 16: force the single-chunk one
    phases &= ~24;
    if (phases < 1 || phases > 7 || schedule == 24 || (schedule != 0 && phases != 7))
        return fail(RC_INVALID_VALUE, "phases must be a mask of 1 (produce), 2 (reduce), 4 (gather); 7 may add 8 or 16");
    const int32_t size = c->size, rank = c->rank;
    if (M < 0 || in_features <= 0 || out_features < 0) return fail(RC_INVALID_VALUE, "negative extent");
    if (in_features % size) return fail(RC_INVALID_VALUE, "in_features %% size != 0");
    if (M % size) return fail(RC_UNSUPPORTED, "M %% size != 0: use the collective-library path");
    const int64_t N = out_features, Kw = in_features / size, Ms = M / size;
    const int64_t lda = input_ld > 0 ? input_ld : Kw;
    if (N % 8 || Kw % 16) return fail(RC_UNSUPPORTED, "needs out_features %% 8 == 0 and (in_features / size) %% 16 == 0");
    if (M > INT32_MAX / 2 || N > INT32_MAX / 2) return fail(RC_UNSUPPORTED, "extent beyond 2^30");
    if (!input || !weight || !scale_M || !scale_N || !output) return fail(RC_INVALID_VALUE, "null pointer argument");
    if (!aligned16(input) || !aligned16(weight) || !aligned16(output) || !aligned16(scale_N) || lda % 16 ||
        (optional_bias && !aligned16(optional_bias)))
        return fail(RC_INVALID_VALUE, "operands must be 16-byte aligned (pointers and leading dimension)");
    if (pplb200_i8i8_row_parallel_p2p_bytes(M, N, size) > c->bytes)
        return fail(RC_INVALID_VALUE, "peer buffer too small for M=%lld N=%lld", (long long)M, (long long)N);
    if (M == 0 || N == 0) return RC_SUCCESS;

    const int64_t recv_off = kFlagBytes + kSlotBytes, staging_off = recv_off + recv_bytes(M, N);
    const Peers pr = peers_of(*c);
    uint32_t* flag_page = reinterpret_cast<uint32_t*>(c->base);
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device);

    // The three steps on the column range [col0, col0 + ncols) of the output (chunk 0 or 1).
    auto produce = [&](cudaStream_t st, int chunk, int64_t col0, int64_t ncols) -> int32_t {
        GemmArgs g;
        g.A = (const int8_t*)input; g.lda = lda; g.B = (const int8_t*)weight + col0 * Kw; g.ldb = Kw;
        g.M = M; g.N = ncols; g.K = Kw; g.mode = EPI_PUSH_I32;
        g.scale_m = nullptr; g.scale_n = nullptr; g.bias = nullptr;
        g.down_m = 0.f; g.down_n = 0.f;
        g.out = nullptr; g.ldc = N;
        g.row_absmax_bits = nullptr;
        for (int r = 0; r < size; ++r) g.push_base[r] = reinterpret_cast<int32_t*>(c->peer[r] + recv_off) + col0;
        g.push_rows = (int32_t)Ms; g.push_rank = rank;
        if (c->sk_ws) { g.sk_ws = c->sk_ws + (chunk ? kSkWsBytes : 0); g.sk_ws_bytes = kSkWsBytes; }
        const int32_t rc = launch_gemm(st, g);
        if (rc != RC_SUCCESS) return rc;
        p2p_signal_kernel<<<1, 32, 0, st>>>(pr, 2 * chunk, chunk == 0 ? 1 : 0);
        return RC_SUCCESS;
    };
    auto reduce = [&](cudaStream_t st, int chunk, int64_t col0, int64_t ncols, int64_t max_blocks) {
        int64_t blocks = (Ms * (ncols >> 3) + 255) / 256;
        if (blocks > max_blocks) blocks = max_blocks;
        p2p_reduce_dequant_kernel<<<(unsigned)blocks, 256, 0, st>>>(
            flag_page, 2 * chunk, size, reinterpret_cast<const int32_t*>(c->base + recv_off), Ms, N, col0, ncols,
            (const half*)scale_M + (int64_t)rank * Ms, (const half*)scale_N, (const half*)optional_bias, down_scale_M,
            down_scale_N, (half*)output + (int64_t)rank * Ms * N, reinterpret_cast<half*>(c->base + staging_off));
        p2p_signal_kernel<<<1, 32, 0, st>>>(pr, 2 * chunk + 1, 0);
    };
    auto gather = [&](cudaStream_t st, int chunk, int64_t col0, int64_t ncols, int64_t max_blocks) {
        if (size == 1) return;
        int64_t blocks = ((Ms * (ncols >> 3) + 255) / 256 * (size - 1) + 3) / 4;
        if (blocks > max_blocks) blocks = max_blocks;
        p2p_gather_kernel<<<(unsigned)blocks, 256, 0, st>>>(pr, 2 * chunk + 1, staging_off, Ms, N, col0, ncols, (half*)output);
    };

    // Two column chunks: the reduction and the row exchange of the first half run on the context's
    // second stream (small grids that share the SMs with the GEMM) under the GEMM of the second half.
    const bool can_chunk = phases == 7 && size > 1 && N % 512 == 0 && M * N >= (int64_t)(4 << 20) &&
                           ((M + 255) / 256) * (N / 512) >= sms / 2;
    // Opt-in only: on 2, 4 and 8 B200s it measured 3 - 16 % slower than the single-chunk schedule (the
    // second stream's kernels slow the GEMM down more than the overlap saves).
    const bool two_chunks = can_chunk && schedule == 8;
    if (two_chunks) {
        const int64_t half_n = N / 2;
        int32_t rc = produce(stream, 0, 0, half_n);
        if (rc != RC_SUCCESS) return rc;
        if (cudaEventRecord(c->fork, stream) != cudaSuccess || cudaStreamWaitEvent(c->side, c->fork, 0) != cudaSuccess)
            return fail(RC_DEVICE_RUNTIME_ERROR, "stream fork failed");
        reduce(c->side, 0, 0, half_n, 2 * sms);
        gather(c->side, 0, 0, half_n, 2 * sms);
        if (cudaEventRecord(c->join, c->side) != cudaSuccess) return fail(RC_DEVICE_RUNTIME_ERROR, "event record failed");
        rc = produce(stream, 1, half_n, half_n);
        if (rc != RC_SUCCESS) return rc;
        reduce(stream, 1, half_n, half_n, 8 * sms);
        gather(stream, 1, half_n, half_n, 8 * sms);
        if (cudaStreamWaitEvent(stream, c->join, 0) != cudaSuccess) return fail(RC_DEVICE_RUNTIME_ERROR, "stream join failed");
        return check_launch("row_parallel_linear_p2p");
    }

    if (phases & 1) {
        const int32_t rc = produce(stream, 0, 0, N);
        if (rc != RC_SUCCESS) return rc;
    }
    if (phases & 2) reduce(stream, 0, 0, N, 8 * sms);
    if (phases & 4) gather(stream, 0, 0, N, 8 * sms);
    return check_launch("row_parallel_linear_p2p");
}

int32_t pplb200_i8i8_column_parallel_linear_p2p(pplb200_stream_t stream_, void* ctx, const void* input, int64_t M,
                                                const void* weight, const void* optional_bias, const void* scale_M,
                                                const void* scale_N, float down_scale_M, float down_scale_N,
                                                int64_t in_features, int64_t out_features, int32_t phases, void* output) {
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    Ctx* c = (Ctx*)ctx;
    if (!c) return fail(RC_INVALID_VALUE, "null context");
    if (!c->connected) return fail(RC_INVALID_VALUE, "context is not connected to its peers");
    if (phases < 1 || phases > 3) return fail(RC_INVALID_VALUE, "phases must be a mask of 1 (produce) and 2 (finish)");
    const int32_t size = c->size, rank = c->rank;
    if (M < 0 || in_features <= 0 || out_features < 0) return fail(RC_INVALID_VALUE, "negative extent");
    if (out_features % size) return fail(RC_INVALID_VALUE, "out_features %% size != 0");
    const int64_t N = out_features, Nw = N / size, K = in_features;
    if (Nw % 8 || K % 16) return fail(RC_UNSUPPORTED, "needs (out_features / size) %% 8 == 0 and in_features %% 16 == 0");
    if (M > INT32_MAX / 2 || N > INT32_MAX / 2) return fail(RC_UNSUPPORTED, "extent beyond 2^30");
    if (!input || !weight || !scale_M || !scale_N || !output) return fail(RC_INVALID_VALUE, "null pointer argument");
    if (!aligned16(input) || !aligned16(weight) || !aligned16(output) || !aligned16(scale_N) ||
        (optional_bias && !aligned16(optional_bias)))
        return fail(RC_INVALID_VALUE, "operands must be 16-byte aligned");
    const int64_t area_off = kFlagBytes + kSlotBytes;
    if (area_off + round_up(M * N * 2, 256) > c->bytes)
        return fail(RC_INVALID_VALUE, "peer buffer too small for a gathered output of M=%lld N=%lld", (long long)M, (long long)N);
    if (M == 0 || N == 0) return RC_SUCCESS;
    const Peers pr = peers_of(*c);
    uint32_t* flag_page = reinterpret_cast<uint32_t*>(c->base);

    if (phases & 1) {
        p2p_wait_consumed_kernel<<<1, 32, 0, stream>>>(flag_page, size);
        GemmArgs g;
        g.A = (const int8_t*)input; g.lda = K; g.B = (const int8_t*)weight; g.ldb = K;
        g.M = M; g.N = Nw; g.K = K; g.mode = EPI_GATHER_F16;
        g.scale_m = (const half*)scale_M; g.scale_n = (const half*)scale_N; g.bias = (const half*)optional_bias;
        g.down_m = down_scale_M; g.down_n = down_scale_N;
        g.out = nullptr; g.ldc = N;
        g.row_absmax_bits = nullptr;
        for (int r = 0; r < size; ++r) g.push_base[r] = reinterpret_cast<int32_t*>(c->peer[r] + area_off);
        g.gather_ranks = size; g.gather_col0 = (int64_t)rank * Nw;
        if (c->sk_ws) { g.sk_ws = c->sk_ws; g.sk_ws_bytes = kSkWsBytes; }
        const int32_t rc = launch_gemm(stream, g);
        if (rc != RC_SUCCESS) return rc;
        p2p_signal_kernel<<<1, 32, 0, stream>>>(pr, kFlagRowGathered, 1, kGatherEpochWord);
    }
    if (phases & 2) {
        int sms = 148;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device);
        const int64_t vecs = M * N / 8;
        int64_t blocks = (vecs + 255) / 256;
        if (blocks > 8 * sms) blocks = 8 * sms;
        p2p_gather_copy_kernel<<<(unsigned)blocks, 256, 0, stream>>>(flag_page, size, reinterpret_cast<const uint4*>(c->base + area_off),
                                                                     vecs, reinterpret_cast<uint4*>(output));
        p2p_signal_kernel<<<1, 32, 0, stream>>>(pr, kFlagRowConsumed, 0, kGatherEpochWord);
    }
    return check_launch("column_parallel_linear_p2p");
}

} // extern "C"

template <int UNITS>
static int32_t launch_p2p_quantize(cudaStream_t stream, const Ctx& c, const half* in, int64_t batch, int64_t dim,
                                   float up_scale, int8_t* q, half* scale, int threads, int publish_only) {
    int per_sm = 0, sms = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, p2p_quantize_rows_kernel<UNITS>, threads, 0) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c.device) != cudaSuccess || per_sm < 1)
        return fail(RC_DEVICE_RUNTIME_ERROR, "occupancy query failed");
    int64_t grid = (int64_t)per_sm * sms; // every CTA resident: none waits for an SM while its row is awaited elsewhere
    if (grid > batch) grid = batch;
    // Cooperative launch: the grid starts only when all of it can be resident at once -- which is what lets every CTA
    // publish all its rows before any CTA waits -- and a grid that could never fit is refused.  An ordinary launch may
    // start part of the grid behind other work; the ranks would then stall each other until their bounded waits ran out.
    Peers pr = peers_of(c);
    void* args[] = {(void*)&in, (void*)&batch, (void*)&dim, (void*)&up_scale, (void*)&q, (void*)&scale, (void*)&pr, (void*)&publish_only};
    const cudaError_t e = cudaLaunchCooperativeKernel((const void*)p2p_quantize_rows_kernel<UNITS>, dim3((unsigned)grid), dim3(threads), args, 0, stream);
    if (e != cudaSuccess) return fail(RC_DEVICE_RUNTIME_ERROR, "sharded quantizer launch failed: %s", cudaGetErrorString(e));
    return check_launch("minmax_quantize_fp16_p2p");
}

extern "C" {

int32_t pplb200_i8i8_minmax_quantize_fp16_p2p(pplb200_stream_t stream_, void* ctx, const void* input, int64_t batch,
                                              int64_t shard_dim, float up_scale, int32_t phases, void* q, void* scale) {
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    Ctx* c = (Ctx*)ctx;
    if (!c) return fail(RC_INVALID_VALUE, "null context");
    if (!c->connected) return fail(RC_INVALID_VALUE, "context is not connected to its peers");
    if (batch < 0 || shard_dim < 0) return fail(RC_INVALID_VALUE, "negative extent");
    if (phases != 1 && phases != 3) return fail(RC_INVALID_VALUE, "phases must be 3 (whole operation) or 1 (publish the shard maxima only)");
    const int publish_only = phases == 1;
    if (batch > kQuantMaxRows) return fail(RC_UNSUPPORTED, "more than %lld rows", (long long)kQuantMaxRows);
    if (shard_dim % 16) return fail(RC_UNSUPPORTED, "shard_dim %% 16 != 0");
    const int64_t units = shard_dim >> 4;
    if (units > (int64_t)QTPB * 8) return fail(RC_UNSUPPORTED, "shard rows longer than %d elements", QTPB * 8 * 16);
    if (batch == 0 || shard_dim == 0) return RC_SUCCESS;
    if (!input || !q || !scale) return fail(RC_INVALID_VALUE, "null pointer argument");
    if (!aligned16(input) || !aligned16(q)) return fail(RC_INVALID_VALUE, "input and output must be 16-byte aligned");
    const int per = (int)((units + QTPB - 1) / QTPB);
    const int bucket = per <= 1 ? 1 : per <= 2 ? 2 : per <= 4 ? 4 : 8;
    int threads = (int)((units + bucket - 1) / bucket);
    threads = (threads + 31) / 32 * 32;
    if (threads > QTPB) threads = QTPB;
    const half* in = (const half*)input;
    switch (bucket) {
    case 1: return launch_p2p_quantize<1>(stream, *c, in, batch, shard_dim, up_scale, (int8_t*)q, (half*)scale, threads, publish_only);
    case 2: return launch_p2p_quantize<2>(stream, *c, in, batch, shard_dim, up_scale, (int8_t*)q, (half*)scale, threads, publish_only);
    case 4: return launch_p2p_quantize<4>(stream, *c, in, batch, shard_dim, up_scale, (int8_t*)q, (half*)scale, threads, publish_only);
    default: return launch_p2p_quantize<8>(stream, *c, in, batch, shard_dim, up_scale, (int8_t*)q, (half*)scale, threads, publish_only);
    }
}

}
