// uint32 inclusive scan for B200: one pass over the data, decoupled look-back
// between tiles.
//
// What it stands in for: `scan_kernel` and its nine device helpers
// (generated/scan_kernel.cu:1-29, generated/scan_warps.cu, get_warp_ends_inclusive.cu,
// naive_scan_warp_ends.cu, write_block_aggregate.cu, write_block_prefix.cu,
// lookback_to_prev_blocks.cu, update_with_new_data_and_writeback.cu,
// get_block_idx_from_global_counter.cu, shfl_up_sync_wrapper.cu) and the host
// glue `get_workspace_size` / `launch_scan` (evals/4090_scan/main.cu:63-86).
//
// How it differs, and why, on a machine whose HBM moves ~6.5 TB/s:
//   * every element is read by one 16-byte load and written by one 16-byte
//     store; the tile lives in registers, not in 64 KB of shared memory, so
//     eight 256-thread CTAs stay resident per SM and keep >100 KB of loads in
//     flight per SM;
//   * the block-level scan is four independent 5-step warp-shuffle scans per
//     thread plus one 8-entry shared-memory hand-off (one __syncthreads), not a
//     9-round Hillis-Steele with a barrier per round;
//   * a tile publishes ONE 64-bit word {state, value}; state says whether value
//     is the tile's own aggregate or its inclusive prefix.  Flag and value
//     travel in one relaxed 64-bit store, so no fence is needed (the reference
//     uses the same packing in BlockInfo, evals/4090_scan/main.cu:21-37, but
//     keeps two words per tile);
//   * look-back is done by a whole warp, 32 predecessors per probe, and every
//     spin is bounded: when it runs out the tile raises an abort flag and a
//     status code instead of hanging the GPU;
//   * tiles take their index from an atomic ticket exactly as the reference
//     does, so a tile's predecessors are always resident or finished.
#include "common.cuh"

namespace prism_b200 {

namespace {

constexpr uint32_t kStateInvalid = 0u;
constexpr uint32_t kStateAggregate = 1u;
constexpr uint32_t kStatePrefix = 2u;
constexpr uint32_t kMaxPolls = 1u << 20;
constexpr size_t kHeaderBytes = 128;  // [0] ticket, [1] abort flag; descriptors follow

template <int THREADS, int VEC>
struct ScanCfg {
    static constexpr int kThreads = THREADS;
    static constexpr int kWarps = THREADS / 32;
    static constexpr int kItems = 4 * VEC;                       // elements per thread
    static constexpr int kWarpElems = 32 * kItems;               // contiguous elements per warp
    static constexpr int kTile = THREADS * kItems;               // elements per CTA
};

__device__ __forceinline__ uint64_t ld_desc(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_desc(uint64_t* p, uint32_t state, uint32_t value) {
    uint64_t v = static_cast<uint64_t>(state) | (static_cast<uint64_t>(value) << 32);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_flag(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ uint32_t warp_sum(uint32_t v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

// TUNING ONLY: per-tile trace of the look-back (windows read, re-polls, timestamps).
#ifdef PRISM_SCAN_TRACE
__device__ unsigned long long g_trace[4 * 65536];
__device__ unsigned int g_trace_polls;
#endif

__device__ __forceinline__ uint64_t poll_desc(const uint64_t* p, uint64_t first, const uint32_t* abort_flag) {
    uint64_t d = first;
    uint32_t polls = 0;
    while (static_cast<uint32_t>(d) == kStateInvalid) {
        if (++polls >= kMaxPolls) break;
        if ((polls & 1023u) == 0u && ld_flag(abort_flag) != 0u) break;
        d = ld_desc(p);
    }
#ifdef PRISM_SCAN_TRACE
    if (polls) atomicAdd(&g_trace_polls, polls);
#endif
    return d;
}

// Sum of the tiles before `tile`, found by walking the records backwards, 32 * NW
// per probe, until one that already carries an inclusive prefix.  The rate at which
// prefixes can propagate is (records per probe) x (tile bytes) per L2 round trip, so
// wide probes and large tiles are what keep this off the critical path.  Executed by
// one full warp.  *failed is set if a bounded poll ran out or an abort was seen.
template <int NW>
__device__ __forceinline__ uint32_t lookback(uint32_t tile, const uint64_t* desc,
                                             const uint32_t* abort_flag, bool* failed) {
    const int lane = threadIdx.x & 31;
    uint32_t exclusive = 0;
    long long idx = static_cast<long long>(tile) - 1 - lane;
    *failed = false;
#ifdef PRISM_SCAN_TRACE
    unsigned long long rounds = 0;
#endif
    while (true) {
#ifdef PRISM_SCAN_TRACE
        ++rounds;
        if (lane == 0 && tile < 65536) g_trace[4 * tile + 2] = rounds;
#endif
        // A slot before tile 0 behaves like a finished tile with prefix 0.
        uint64_t d[NW];
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const long long i = idx - 32 * w;
            d[w] = i >= 0 ? ld_desc(desc + i) : static_cast<uint64_t>(kStatePrefix);
        }
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const long long i = idx - 32 * w;
            if (i >= 0) d[w] = poll_desc(desc + i, d[w], abort_flag);
            const uint32_t state = static_cast<uint32_t>(d[w]);
            const uint32_t value = static_cast<uint32_t>(d[w] >> 32);
            if (!__all_sync(0xffffffffu, state != kStateInvalid)) {
                *failed = true;
                return exclusive;
            }
            const unsigned has_prefix = __ballot_sync(0xffffffffu, state == kStatePrefix);
            if (has_prefix) {
                const int first = __ffs(has_prefix) - 1;  // nearest predecessor with a prefix
                exclusive += warp_sum(lane <= first ? value : 0u);
                return exclusive;
            }
            exclusive += warp_sum(value);
        }
        idx -= 32 * NW;
    }
}

template <int THREADS, int VEC, int NW, bool SEEDED, bool TICKET = true, bool LOOKBACK = true>
__device__ __forceinline__ void scan_tile_body(uint32_t n, uint32_t* x, uint32_t* header,
                                               uint64_t* desc, const uint32_t* totals, int rank) {
    using Cfg = ScanCfg<THREADS, VEC>;
    constexpr int kScanWarps = Cfg::kWarps;
    __shared__ uint32_t s_tile;
    __shared__ uint32_t s_warp_total[kScanWarps];
    __shared__ uint32_t s_prefix;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;

    if (TICKET) {
        if (tid == 0) s_tile = atomicAdd(header, 1u);
        __syncthreads();
    }
    const uint32_t tile = TICKET ? s_tile : blockIdx.x;
    const unsigned long long base =
        static_cast<unsigned long long>(tile) * Cfg::kTile + static_cast<unsigned long long>(warp) * Cfg::kWarpElems;
    const bool full_tile = static_cast<unsigned long long>(tile) * Cfg::kTile + Cfg::kTile <= n;

    uint4 v[VEC];
    if (full_tile) {
#pragma unroll
        for (int j = 0; j < VEC; ++j)
            v[j] = __ldcg(reinterpret_cast<const uint4*>(x + base + j * 128 + lane * 4));
    } else {
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            const unsigned long long e = base + j * 128 + lane * 4;
            v[j].x = (e + 0 < n) ? x[e + 0] : 0u;
            v[j].y = (e + 1 < n) ? x[e + 1] : 0u;
            v[j].z = (e + 2 < n) ? x[e + 2] : 0u;
            v[j].w = (e + 3 < n) ? x[e + 3] : 0u;
        }
    }

    // Inside each 16-byte group, then across the 32 lanes of each of the VEC chunks.
    uint32_t sum[VEC], inc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
        v[j].y += v[j].x;
        v[j].z += v[j].y;
        v[j].w += v[j].z;
        sum[j] = v[j].w;
        inc[j] = sum[j];
    }
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            const uint32_t up = __shfl_up_sync(0xffffffffu, inc[j], d);
            if (lane >= d) inc[j] += up;
        }
    }
    // Offset of each chunk inside the warp, and the warp's total.
    uint32_t chunk_off = 0;
    uint32_t excl[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
        excl[j] = chunk_off + inc[j] - sum[j];
        chunk_off += __shfl_sync(0xffffffffu, inc[j], 31);
    }
    if (lane == 0) s_warp_total[warp] = chunk_off;
    __syncthreads();

    uint32_t warp_off = 0, aggregate = 0;
#pragma unroll
    for (int w = 0; w < kScanWarps; ++w) {
        const uint32_t t = s_warp_total[w];
        if (w < warp) warp_off += t;
        aggregate += t;
    }

    if (warp == 0) {
        uint32_t exclusive = 0;
        if (tile == 0) {
            if (SEEDED) {
                for (int r = 0; r < rank; ++r) exclusive += totals[r];
            }
            if (lane == 0) st_desc(desc, kStatePrefix, exclusive + aggregate);
        } else {
            if (lane == 0) st_desc(desc + tile, kStateAggregate, aggregate);
#ifdef PRISM_SCAN_TRACE
            if (lane == 0 && tile < 65536) g_trace[4 * tile + 0] = global_timer_ns();
#endif
            bool failed;
            exclusive = LOOKBACK ? lookback<NW>(tile, desc, header + 1, &failed) : 0u;
            if (!LOOKBACK) failed = false;
#ifdef PRISM_SCAN_TRACE
            if (lane == 0 && tile < 65536) g_trace[4 * tile + 1] = global_timer_ns();
#endif
            if (lane == 0) {
                if (failed) {
                    atomicExch(header + 1, 1u);
                    raise_device_status(DEV_SCAN_LOOKBACK_TIMEOUT);
                }
                st_desc(desc + tile, kStatePrefix, exclusive + aggregate);
            }
        }
        if (lane == 0) s_prefix = exclusive;
    }
    __syncthreads();
    const uint32_t add = s_prefix + warp_off;

    if (full_tile) {
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            const uint32_t a = add + excl[j];
            v[j].x += a; v[j].y += a; v[j].z += a; v[j].w += a;
            __stcg(reinterpret_cast<uint4*>(x + base + j * 128 + lane * 4), v[j]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            const uint32_t a = add + excl[j];
            const unsigned long long e = base + j * 128 + lane * 4;
            if (e + 0 < n) x[e + 0] = v[j].x + a;
            if (e + 1 < n) x[e + 1] = v[j].y + a;
            if (e + 2 < n) x[e + 2] = v[j].z + a;
            if (e + 3 < n) x[e + 3] = v[j].w + a;
        }
    }
}

// Tile geometry: threads per CTA, 16-byte vectors per thread, look-back probes of 32 * NW records.
constexpr int kThreads = 256;
constexpr int kVec = 4;
constexpr int kNW = 1;
constexpr int kMinTile = 4096;  // the workspace is sized for the smallest tile any variant uses

}  // namespace

// Same parameter list as the reference entry point (generated/scan_kernel.cu:1):
// n elements, data in place, the ticket counter, the per-tile records.  Here the
// counter word is followed by an abort flag and a record is one 64-bit word.
__global__ void __launch_bounds__(kThreads)
scan_kernel(uint32_t n, uint32_t* x, uint32_t* block_idx_counter, int* block_infos) {
    scan_tile_body<kThreads, kVec, kNW, false>(n, x, block_idx_counter, reinterpret_cast<uint64_t*>(block_infos),
                                               nullptr, 0);
}

// Sharded form: tile 0 starts from totals[0] + ... + totals[rank-1].
__global__ void __launch_bounds__(kThreads)
scan_kernel_seeded(uint32_t n, uint32_t* x, uint32_t* block_idx_counter, int* block_infos,
                   const uint32_t* totals, int rank) {
    scan_tile_body<kThreads, kVec, kNW, true>(n, x, block_idx_counter, reinterpret_cast<uint64_t*>(block_infos),
                                              totals, rank);
}

// TUNING ONLY: other geometries, selected with PRISM_B200_SCAN_VARIANT.
template <int THREADS, int VEC, int NW, bool TICKET = true, bool LOOKBACK = true>
__global__ void __launch_bounds__(THREADS)
scan_kernel_var(uint32_t n, uint32_t* x, uint32_t* block_idx_counter, int* block_infos, const uint32_t* totals,
                int rank) {
    scan_tile_body<THREADS, VEC, NW, true, TICKET, LOOKBACK>(n, x, block_idx_counter,
                                                             reinterpret_cast<uint64_t*>(block_infos), totals, rank);
}

__global__ void __launch_bounds__(256) reduce_u32_kernel(size_t n, const uint32_t* x, uint32_t* total) {
    __shared__ uint32_t s_part[8];
    uint32_t acc = 0;
    const size_t n4 = n / 4;
    const uint4* x4 = reinterpret_cast<const uint4*>(x);
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    // Four independent 16-byte loads in flight per thread.
    for (; i + 3 * stride < n4; i += 4 * stride) {
        const uint4 a = __ldcg(x4 + i), b = __ldcg(x4 + i + stride), c = __ldcg(x4 + i + 2 * stride),
                    d = __ldcg(x4 + i + 3 * stride);
        acc += (a.x + a.y) + (a.z + a.w) + (b.x + b.y) + (b.z + b.w) + (c.x + c.y) + (c.z + c.w) + (d.x + d.y) +
               (d.z + d.w);
    }
    for (; i < n4; i += stride) {
        const uint4 a = __ldcg(x4 + i);
        acc += (a.x + a.y) + (a.z + a.w);
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) acc += x[n4 * 4 + threadIdx.x];
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x < 32) {
        uint32_t v = threadIdx.x < 8 ? s_part[threadIdx.x] : 0u;
        v = warp_sum(v);
        if (threadIdx.x == 0) atomicAdd(total, v);
    }
}

__global__ void __launch_bounds__(256) add_carry_kernel(size_t n, uint32_t* x, const uint32_t* totals, int rank) {
    uint32_t carry = 0;
    for (int r = 0; r < rank; ++r) carry += totals[r];
    const size_t n4 = n / 4;
    uint4* x4 = reinterpret_cast<uint4*>(x);
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        uint4 a = __ldcg(x4 + i);
        a.x += carry; a.y += carry; a.z += carry; a.w += carry;
        __stcg(x4 + i, a);
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) x[n4 * 4 + threadIdx.x] += carry;
}

namespace {

size_t scan_tiles(size_t n) { return (n + kMinTile - 1) / kMinTile; }

using VarKernel = void (*)(uint32_t, uint32_t*, uint32_t*, int*, const uint32_t*, int);
struct Variant { VarKernel k; int threads; int tile; };
#define PRISM_VARIANT(T, V, W) Variant{scan_kernel_var<T, V, W>, T, T * 4 * V}
const Variant kVariants[] = {
    PRISM_VARIANT(256, 4, 1),   // 0
    PRISM_VARIANT(256, 4, 2),   // 1
    PRISM_VARIANT(512, 4, 1),   // 2
    PRISM_VARIANT(512, 8, 1),   // 3
    PRISM_VARIANT(512, 8, 2),   // 4
    PRISM_VARIANT(256, 8, 2),   // 5
    PRISM_VARIANT(1024, 4, 2),  // 6
    PRISM_VARIANT(256, 16, 2),  // 7
    PRISM_VARIANT(1024, 4, 1),  // 8
    PRISM_VARIANT(512, 8, 4),   // 9
    Variant{scan_kernel_var<512, 8, 1, false, true>, 512, 16384},   // 10 no ticket
    Variant{scan_kernel_var<512, 8, 1, true, false>, 512, 16384},   // 11 no look-back (wrong results)
    Variant{scan_kernel_var<512, 8, 1, false, false>, 512, 16384},  // 12 neither
    Variant{scan_kernel_var<256, 4, 1, false, true>, 256, 4096},    // 13 no ticket
    Variant{scan_kernel_var<256, 4, 1, false, false>, 256, 4096},   // 14 neither
    Variant{scan_kernel_var<256, 8, 1, false, true>, 256, 8192},    // 15 no ticket
};
int scan_variant() {
    static int v = -2;
    if (v == -2) {
        const char* e = getenv("PRISM_B200_SCAN_VARIANT");
        v = e ? atoi(e) : -1;
        if (v >= static_cast<int>(sizeof(kVariants) / sizeof(kVariants[0]))) v = -1;
    }
    return v;
}

int scan_launch(size_t n, uint32_t* x, void* workspace, const uint32_t* totals, int rank, bool seeded,
                cudaStream_t stream) {
    if (n == 0) return PRISM_B200_OK;
    if (!x || !workspace) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "scan: null pointer");
    if (n >= (1ull << 32)) return set_error(PRISM_B200_ERR_TOO_LARGE, "scan: n=%zu must be below 2^32", n);
    if (reinterpret_cast<uintptr_t>(x) & 15u) return set_error(PRISM_B200_ERR_MISALIGNED, "scan: x not 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(workspace) & 15u)
        return set_error(PRISM_B200_ERR_MISALIGNED, "scan: workspace not 16-byte aligned");
    if (seeded && (rank < 0 || (rank > 0 && !totals)))
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "scan_seeded: bad rank/totals");
    if (int rc = bind_status_word()) return rc;

    const int var = scan_variant();
    const int tile_elems = var >= 0 ? kVariants[var].tile : ScanCfg<kThreads, kVec>::kTile;
    const uint32_t tiles = static_cast<uint32_t>((n + tile_elems - 1) / tile_elems);
    uint32_t* header = static_cast<uint32_t*>(workspace);
    uint64_t* desc = reinterpret_cast<uint64_t*>(static_cast<char*>(workspace) + kHeaderBytes);
    // One memset re-arms ticket, abort flag and every record (the reference
    // issues two, evals/4090_scan/main.cu:81-82).
    PRISM_CUDA_TRY(cudaMemsetAsync(workspace, 0, kHeaderBytes + static_cast<size_t>(tiles) * sizeof(uint64_t), stream));
    if (var >= 0)
        kVariants[var].k<<<tiles, kVariants[var].threads, 0, stream>>>(static_cast<uint32_t>(n), x, header,
                                                                       reinterpret_cast<int*>(desc), totals,
                                                                       seeded ? rank : 0);
    else if (seeded)
        scan_kernel_seeded<<<tiles, kThreads, 0, stream>>>(static_cast<uint32_t>(n), x, header,
                                                            reinterpret_cast<int*>(desc), totals, rank);
    else
        scan_kernel<<<tiles, kThreads, 0, stream>>>(static_cast<uint32_t>(n), x, header,
                                                     reinterpret_cast<int*>(desc));
    PRISM_CUDA_TRY(cudaGetLastError());
    count_launch();
    return PRISM_B200_OK;
}

unsigned streaming_grid(size_t n4) {
    size_t blocks = (n4 + 256 * 4 - 1) / (256 * 4);
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 8) blocks = 148 * 8;
    return static_cast<unsigned>(blocks);
}

}  // namespace
}  // namespace prism_b200

using namespace prism_b200;

// ---------------------------------------------------------------------------
// Scan for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc on the path that runs the
// scan: a plugin that is handed device buffers by its host application and is
// forbidden to grow the process's memory footprint, a real-time loop that may
// not block on the allocator, code running after the application has handed all
// remaining device memory to its own pool.  prism_b200_scan needs caller-provided
// scratch, which such callers have nowhere to get from.  This entry point keeps
// the scratch inside the library image instead: a fixed array in device memory
// that exists on every GPU that loads the library, from load until exit.
// ---------------------------------------------------------------------------
namespace prism_b200 {
namespace {
constexpr size_t kStaticMaxN = 1ull << 28;  // elements (1 GiB of data)
constexpr size_t kStaticScratchBytes = kHeaderBytes + (kStaticMaxN / kMinTile) * sizeof(uint64_t);  // 524,416 B
}  // namespace
}  // namespace prism_b200

// In host code this name is only a handle for the runtime; the device address
// comes from cudaGetSymbolAddress (static_scratch_address below).
static __device__ __align__(256) unsigned char g_static_scan_scratch[prism_b200::kStaticScratchBytes];

namespace prism_b200 {
namespace {
void* g_static_scratch_addr[64] = {};

// Device address of the built-in scratch on the current device, looked up once per device.
int static_scratch_address(void** out) {
    int dev = 0;
    PRISM_CUDA_TRY(cudaGetDevice(&dev));
    const bool cacheable = dev >= 0 && dev < 64;
    if (cacheable && g_static_scratch_addr[dev]) {
        *out = g_static_scratch_addr[dev];
        return PRISM_B200_OK;
    }
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scan_scratch);
    if (e != cudaSuccess) return cuda_failed(e, "cudaGetSymbolAddress(built-in scan scratch)");
    if (!p) return set_error(PRISM_B200_ERR_CUDA, "built-in scan scratch has no device address");
    if (cacheable) g_static_scratch_addr[dev] = p;
    *out = p;
    return PRISM_B200_OK;
}
}  // namespace
}  // namespace prism_b200

extern "C" int prism_b200_scan_static(size_t n, uint32_t* x, void* stream) {
    if (n == 0) return PRISM_B200_OK;
    if (!x) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "scan_static: null pointer");
    if (n > kStaticMaxN)
        return set_error(PRISM_B200_ERR_TOO_LARGE,
                         "scan_static: n=%zu exceeds the built-in scratch (at most %zu elements); use prism_b200_scan "
                         "with caller-provided scratch",
                         n, static_cast<size_t>(kStaticMaxN));
    if (reinterpret_cast<uintptr_t>(x) & 15u)
        return set_error(PRISM_B200_ERR_MISALIGNED, "scan_static: x not 16-byte aligned");
    void* scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    constexpr int tile_elems = ScanCfg<kThreads, kVec>::kTile;
    const uint32_t tiles = static_cast<uint32_t>((n + tile_elems - 1) / tile_elems);
    uint32_t* header = static_cast<uint32_t*>(scratch);
    uint64_t* desc = reinterpret_cast<uint64_t*>(static_cast<char*>(scratch) + kHeaderBytes);
    // The array still holds the previous call's ticket, abort flag and records.
    PRISM_CUDA_TRY(cudaMemsetAsync(scratch, 0, kHeaderBytes + static_cast<size_t>(tiles) * sizeof(uint64_t), s));
    scan_kernel<<<tiles, kThreads, 0, s>>>(static_cast<uint32_t>(n), x, header, reinterpret_cast<int*>(desc));
    PRISM_CUDA_TRY(cudaGetLastError());
    count_launch();
    return PRISM_B200_OK;
}

#ifdef PRISM_SCAN_TRACE
extern "C" int prism_b200_scan_trace(unsigned long long* out, unsigned int* polls) {
    cudaMemcpyFromSymbol(out, g_trace, sizeof(unsigned long long) * 4 * 65536);
    cudaMemcpyFromSymbol(polls, g_trace_polls, 4);
    unsigned int z = 0;
    cudaMemcpyToSymbol(g_trace_polls, &z, 4);
    return 0;
}
#endif

extern "C" int prism_b200_scan_workspace_size(size_t n, size_t* bytes) {
    if (!bytes) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "scan_workspace_size: null bytes");
    if (n >= (1ull << 32)) return set_error(PRISM_B200_ERR_TOO_LARGE, "scan: n=%zu must be below 2^32", n);
    *bytes = kHeaderBytes + scan_tiles(n) * sizeof(uint64_t);
    return PRISM_B200_OK;
}

extern "C" int prism_b200_scan(size_t n, uint32_t* x, void* workspace, void* stream) {
    return scan_launch(n, x, workspace, nullptr, 0, false, static_cast<cudaStream_t>(stream));
}

extern "C" int prism_b200_scan_seeded(size_t n, uint32_t* x, void* workspace, const uint32_t* totals, int rank,
                                      void* stream) {
    return scan_launch(n, x, workspace, totals, rank, true, static_cast<cudaStream_t>(stream));
}

extern "C" int prism_b200_reduce_u32(size_t n, const uint32_t* x, uint32_t* total, void* stream) {
    if (!total || (n && !x)) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "reduce_u32: null pointer");
    if (reinterpret_cast<uintptr_t>(x) & 15u)
        return set_error(PRISM_B200_ERR_MISALIGNED, "reduce_u32: x not 16-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    PRISM_CUDA_TRY(cudaMemsetAsync(total, 0, sizeof(uint32_t), s));
    if (n == 0) return PRISM_B200_OK;
    reduce_u32_kernel<<<streaming_grid(n / 4), 256, 0, s>>>(n, x, total);
    PRISM_CUDA_TRY(cudaGetLastError());
    count_launch();
    return PRISM_B200_OK;
}

extern "C" int prism_b200_scan_add_carry(size_t n, uint32_t* x, const uint32_t* totals, int rank, void* stream) {
    if (rank < 0 || (n && !x) || (rank > 0 && !totals))
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "scan_add_carry: bad argument");
    if (reinterpret_cast<uintptr_t>(x) & 15u)
        return set_error(PRISM_B200_ERR_MISALIGNED, "scan_add_carry: x not 16-byte aligned");
    if (n == 0 || rank == 0) return PRISM_B200_OK;
    add_carry_kernel<<<streaming_grid(n / 4), 256, 0, static_cast<cudaStream_t>(stream)>>>(n, x, totals, rank);
    PRISM_CUDA_TRY(cudaGetLastError());
    count_launch();
    return PRISM_B200_OK;
}
