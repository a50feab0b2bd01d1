// uint32 inclusive scan for B200: one pass over the data, decoupled look-back
// between tiles, tiles parked in shared memory while their prefix is in flight.
//
// What it stands in for: `scan_kernel` and its nine device helpers
// (generated/scan_kernel.cu:1-29, generated/scan_warps.cu, get_warp_ends_inclusive.cu,
// naive_scan_warp_ends.cu, write_block_aggregate.cu, write_block_prefix.cu,
// lookback_to_prev_blocks.cu, update_with_new_data_and_writeback.cu,
// get_block_idx_from_global_counter.cu, shfl_up_sync_wrapper.cu) and the host
// glue `get_workspace_size` / `launch_scan` (evals/4090_scan/main.cu:63-86).
//
// Why it is shaped the way it is.  A one-tile-per-CTA scan that keeps its tile in
// registers streams at HBM speed on B200 if the look-back is taken out (6.8 TB/s
// measured) but reaches 2.9-3.8 TB/s with it: every tile waits ~5 us for its
// predecessors, mostly for aggregates that are published late, and while it
// waits its data occupies registers that the SM needs to keep loads in flight.
// So here a CTA is persistent and owns a ring of S 16 KB slots in shared memory:
//   producer warp   draws a ticket (the reference's atomic tile counter), bulk-copies
//                   that tile into the next free slot with cp.async.bulk; completion
//                   is counted on the slot's "full" mbarrier;
//   8 scan warps    phase A when a slot fills: slot -> registers, tile-local scan
//                   (serial over 4 elements, four independent 5-step warp-shuffle
//                   scans per lane, one 8-entry hand-off between warps), scanned
//                   values back into the slot, tile aggregate published;
//                   phase B, once the tile's prefix is known: slot -> registers, add the
//                   exclusive prefix, 16-byte stores to global memory, slot released;
//   look-back warp  resolves the exclusive prefix of the CTA's tiles in order, 32
//                   predecessor records per probe, and publishes inclusive prefixes.
// Between A and B a tile costs only shared memory, so loads keep flowing.
//
// A tile publishes ONE 64-bit record {state, value}, alone in a 32-byte sector; state says whether value is
// the tile's own aggregate or its inclusive prefix.  Flag and value travel in one
// relaxed 64-bit store, so they cannot tear and no fence is needed (the reference
// packs the same way in BlockInfo, evals/4090_scan/main.cu:21-37, but keeps two
// words per tile).
//
// No-deadlock argument, as in the reference: a tile only ever waits for tiles with
// smaller tickets; a ticket is drawn only when a slot is free, so the load of a
// ticketed tile never waits on anything, and the CTA holding the smallest unresolved
// ticket can always finish it.  CTAs need not be co-resident.  Every wait is bounded
// all the same: one that runs out raises an abort flag and a status code, all roles
// unwind and the kernel returns.
#include "common.cuh"

#include <mutex>
#include <type_traits>

namespace prism_b200 {

namespace {

constexpr uint32_t kStateInvalid = 0u;
constexpr uint32_t kStateAggregate = 1u;
constexpr uint32_t kStatePrefix = 2u;
constexpr size_t kHeaderBytes = 128;  // [0] ticket, [1] abort flag; the records follow
// 64-bit words between consecutive tiles' records: one 32-byte sector per record.  Packed records
// (16 to a 128-byte line) cost 11 % of the throughput: up to 32 look-back warps poll each record
// and the polls of neighbouring records then queue on the same sector.
constexpr int kRecStride = 4;

constexpr int kScanThreads = 256;               // 8 scan warps
constexpr int kLookbackWarps = 1;               // warp q resolves ring items q, q + kLookbackWarps, ... (more measured slower)
constexpr int kThreads = kScanThreads + 32 + 32 * kLookbackWarps;  // + producer warp + look-back warps
constexpr int kVecs = 4;                        // 16-byte vectors per lane
constexpr int kTile = kScanThreads * 4 * kVecs; // 4096 elements = 16 KB
constexpr int kSlots = 4;                       // ring depth: 3 CTAs of 64 KB per SM (3, 5 and 6 measured slower)
constexpr uint32_t kSentinel = 0xFFFFFFFFu;

constexpr size_t kSlotBytes = static_cast<size_t>(kTile) * 4;
// slots, 4 barriers per slot, aggregate and prefix per slot and 2 x 8 warp totals (8 bytes each, whatever the
// element width), tile index per slot, four control words
constexpr size_t kSmemBytes = kSlots * kSlotBytes + 4 * kSlots * 8 + 2 * kSlots * 8 + 2 * 8 * 8 + kSlots * 4 + 4 * 4;

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

// Element arithmetic on 32- or 64-bit containers: wrap-around integer adds, or fp32 adds on the bit
// patterns (F32, 32-bit only).  The all-zero pattern is the identity of each.
using u64 = unsigned long long;
template <bool F32, typename E>
__device__ __forceinline__ E eadd(E a, E b) {
    if constexpr (F32) return __float_as_uint(__fadd_rn(__uint_as_float(a), __uint_as_float(b)));
    else return a + b;
}

template <bool F32 = false, typename E = uint32_t>
__device__ __forceinline__ E warp_sum(E v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = eadd<F32, E>(v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
}

// A tile's record.  32-bit values: ONE 64-bit word {state, value}.  64-bit values: TWO such words in the tile's
// sector, {state, low half} and {state, high half}; each is written and read whole, and a reader takes the pair
// only when both carry the same state (a word is written once per state, so equal states mean one publication).
template <typename E>
__device__ __forceinline__ void rec_publish(uint64_t* rec, uint32_t state, E value) {
    if constexpr (sizeof(E) == 4) {
        st_desc(rec, state, value);
    } else {
        st_desc(rec, state, static_cast<uint32_t>(value));
        st_desc(rec + 1, state, static_cast<uint32_t>(value >> 32));
    }
}
template <typename E>
__device__ __forceinline__ uint32_t rec_read(const uint64_t* rec, E* value) {
    if constexpr (sizeof(E) == 4) {
        const uint64_t d = ld_desc(rec);
        *value = static_cast<uint32_t>(d >> 32);
        return static_cast<uint32_t>(d);
    } else {
        const uint64_t lo = ld_desc(rec), hi = ld_desc(rec + 1);
        *value = (lo >> 32) | (hi & 0xFFFFFFFF00000000ull);
        return static_cast<uint32_t>(lo) == static_cast<uint32_t>(hi) ? static_cast<uint32_t>(lo) : kStateInvalid;
    }
}

__device__ __forceinline__ void bulk_load_tile(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Sum of the tiles before `tile`, found by walking the records backwards 32 at a
// time until one that already carries an inclusive prefix (the job of the reference's
// lookback_to_prev_blocks, generated/lookback_to_prev_blocks.cu:8-25, done by a warp
// instead of a thread and with bounded spins).  *failed is set if a poll ran out or
// an abort was seen.
template <bool F32, typename E>
__device__ __forceinline__ E lookback(uint32_t tile, const uint64_t* desc, const uint32_t* abort_flag,
                                      unsigned long long limit_ns, bool* failed) {
    const int lane = threadIdx.x & 31;
    E exclusive = 0;
    long long idx = static_cast<long long>(tile) - 1 - lane;
    *failed = false;
    while (true) {
        // A slot before tile 0 behaves like a finished tile with prefix 0.
        uint32_t state = kStatePrefix;
        E value = 0;
        if (idx >= 0) {
            uint32_t polls = 0;
            unsigned long long t0 = 0;
            state = rec_read<E>(desc + idx * kRecStride, &value);
            while (state == kStateInvalid) {
                if ((++polls & 1023u) == 0u) {
                    if (t0 == 0) t0 = global_timer_ns();
                    if (ld_flag(abort_flag) != 0u || global_timer_ns() - t0 > limit_ns) break;
                }
                state = rec_read<E>(desc + idx * kRecStride, &value);
            }
        }
        if (!__all_sync(0xffffffffu, state != kStateInvalid)) {
            *failed = true;
            return exclusive;
        }
        const unsigned has_prefix = __ballot_sync(0xffffffffu, state == kStatePrefix);
        if (has_prefix) {
            const int first = __ffs(has_prefix) - 1;  // nearest predecessor with a prefix
            exclusive = eadd<F32, E>(exclusive, warp_sum<F32, E>(lane <= first ? value : E(0)));
            return exclusive;
        }
        exclusive = eadd<F32, E>(exclusive, warp_sum<F32, E>(value));
        idx -= 32;
    }
}

// Where tile 0's exclusive prefix comes from.
//   kSeedNone    0
//   kSeedTotals  totals[0] + ... + totals[rank-1], an array in this GPU's memory (filled by an all-gather)
//   kSeedPeers   the same sum, but each total arrives as a {epoch, total} word that the owning rank stores
//                straight into this GPU's memory over NVLink; the look-back warp waits (bounded) until every
//                rank's word carries this call's epoch
enum { kSeedNone = 0, kSeedTotals = 1, kSeedPeers = 2, kSeedNoneF32 = 3 /* host-side selector of the fp32 kernel */ };

__device__ __forceinline__ uint64_t ld_sys_u64(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_sys_u64(uint64_t* p, uint64_t v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// What the sharded kernel needs beyond the plain scan's arguments.
struct ShardArgs {
    const uint64_t* slots;         // this rank's 2 * world words, written by every rank
    uint64_t* const* peer_slots;   // base address of every rank's word array (device array of `world` pointers)
    int rank, world;
    uint32_t epoch;                // non-zero, the same on every rank, changes from call to call
    uint32_t phases;               // kPhaseReduce | kPhaseScan
    unsigned long long wait_ns;    // longest wait for the other ranks' words
};
enum : uint32_t { kPhaseReduce = 1u, kPhaseScan = 2u };

// Header words of the scratch: [0] scan ticket, [1] abort flag, and for the sharded kernel
// [2] reduce ticket, [3] reduce slices finished, [4] running total of the chunk.
constexpr uint32_t kSliceElems = 1u << 15;   // elements per reduce ticket (128 KB)

// First phase of the sharded kernel: the CTAs draw slices of the chunk, LAST slice first (what is still
// in L2 afterwards is then the part the scan reads first), add them up, and whoever finishes the last
// slice stores {epoch, total} into every rank's word array, one 64-bit system-scope store each, over
// NVLink for the peers.  Slices are handed out by ticket, so a CTA that is not resident yet holds
// nobody up.  All threads of the CTA take part; `s_ticket` (two words) and `s_part` are shared-memory scratch.
__device__ __forceinline__ void reduce_and_publish(uint32_t n, const uint32_t* src, uint32_t* header, const ShardArgs& sh,
                                                   volatile uint32_t* s_ticket, volatile uint32_t* s_part) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t slices = static_cast<uint32_t>((static_cast<unsigned long long>(n) + kSliceElems - 1) / kSliceElems);
    auto publish = [&](uint32_t total) {
        const uint64_t w = static_cast<uint64_t>(sh.epoch) | (static_cast<uint64_t>(total) << 32);
        for (int p = 0; p < sh.world; ++p) st_sys_u64(sh.peer_slots[p] + (sh.epoch & 1u) * sh.world + sh.rank, w);
    };
    if (slices == 0) {   // an empty chunk still announces itself: the others wait for every rank's word
        if (blockIdx.x == 0 && tid == 0) publish(0u);
        return;
    }
    // The next ticket is drawn while the current slice is being read, and the partial sums stay in registers
    // until the CTA has no more slices: one barrier per slice, one block-wide sum and two atomics per CTA.
    uint32_t acc = 0, mine = 0;
    if (tid == 0) s_ticket[0] = atomicAdd(header + 2, 1u);
    __syncthreads();
    for (uint32_t k = 0;; ++k) {
        const uint32_t t = s_ticket[k & 1u];
        if (t >= slices) break;
        if (tid == 0) s_ticket[(k + 1u) & 1u] = atomicAdd(header + 2, 1u);
        const unsigned long long lo = static_cast<unsigned long long>(slices - 1 - t) * kSliceElems;
        const uint32_t cnt = n - lo < kSliceElems ? static_cast<uint32_t>(n - lo) : kSliceElems;
        const uint4* p4 = reinterpret_cast<const uint4*>(src + lo);
        const uint32_t nv = cnt / 4;
        uint32_t v = tid;
        for (; v + 3 * kThreads < nv; v += 4 * kThreads) {
            const uint4 a = __ldcg(p4 + v), b = __ldcg(p4 + v + kThreads), c = __ldcg(p4 + v + 2 * kThreads),
                        d = __ldcg(p4 + v + 3 * kThreads);
            acc += (a.x + a.y) + (a.z + a.w) + (b.x + b.y) + (b.z + b.w) + (c.x + c.y) + (c.z + c.w) + (d.x + d.y) +
                   (d.z + d.w);
        }
        for (; v < nv; v += kThreads) {
            const uint4 a = __ldcg(p4 + v);
            acc += (a.x + a.y) + (a.z + a.w);
        }
        if (static_cast<uint32_t>(tid) < (cnt & 3u)) acc += src[lo + nv * 4 + tid];
        ++mine;
        __syncthreads();   // the next ticket is in place, and everybody has read this one
    }
    acc = warp_sum(acc);
    if (lane == 0) s_part[warp] = acc;
    __syncthreads();
    if (tid == 0 && mine > 0) {
        uint32_t tot = 0;
        for (int w = 0; w < kThreads / 32; ++w) tot += s_part[w];
        atomicAdd(header + 4, tot);
        __threadfence();
        if (atomicAdd(header + 3, mine) + mine == slices) {   // every slice has been added
            __threadfence();
            publish(atomicAdd(header + 4, 0u));
        }
    }
}

// Waits (at most sh.wait_ns) until every rank's word in this rank's array carries this call's epoch and
// returns the sum of the lower ranks' totals.  Every rank's word is awaited, not only the lower ones:
// that a rank has seen all words of epoch e is what allows the others to overwrite that half of the
// array at epoch e + 2, and this rank's own word says that its reduce phase has read the whole chunk,
// which the scan is about to overwrite.  Called by one whole warp; lane r watches rank r.
__device__ __forceinline__ uint32_t wait_peer_words(const ShardArgs& sh, volatile uint32_t* abort_flag, bool* failed) {
    const int lane = threadIdx.x & 31;
    const uint64_t* words = sh.slots + (sh.epoch & 1u) * sh.world;
    uint64_t w = static_cast<uint64_t>(sh.epoch);
    if (lane < sh.world) {
        const unsigned long long t0 = global_timer_ns();
        w = ld_sys_u64(words + lane);
        for (uint32_t spin = 1; static_cast<uint32_t>(w) != sh.epoch; ++spin) {
            if ((spin & 63u) == 0u && (*abort_flag || global_timer_ns() - t0 > sh.wait_ns)) break;
            __nanosleep(100);
            w = ld_sys_u64(words + lane);
        }
    }
    *failed = !__all_sync(0xffffffffu, static_cast<uint32_t>(w) == sh.epoch);
    return warp_sum(lane < sh.rank ? static_cast<uint32_t>(w >> 32) : 0u);
}

// `src` is read, `x` is written (the same pointer for the in-place entry points).  EXCL shifts the
// result by one element: out[i] = in[0] + ... + in[i-1], out[0] = the seed.  I64: the elements are
// 64-bit integers (wrap-around adds); a tile is then 2048 elements, still 16 KB, and a 16-byte vector
// holds two of them.  `n` counts elements.
template <int SEED, bool F32 = false, bool EXCL = false, bool I64 = false>
__device__ __forceinline__ void scan_body(uint32_t n, const void* src_v, void* x_v, uint32_t* header, uint64_t* desc,
                                          const void* seed_src, int rank, const ShardArgs* shard = nullptr) {
    static_assert(!(F32 || I64) || SEED == kSeedNone, "the sharded forms are uint32 only");
    static_assert(!(F32 && I64), "fp32 adds are 32-bit");
    using E = typename std::conditional<I64, u64, uint32_t>::type;
    constexpr int EPV = 16 / static_cast<int>(sizeof(E));        // elements per 16-byte vector
    constexpr uint32_t TILE = kTile * 4 / sizeof(E);             // elements per tile
    constexpr int CHUNK = 32 * EPV;                              // elements a warp covers with one vector per lane
    const E* src = static_cast<const E*>(src_v);
    E* x = static_cast<E*>(x_v);
    // Longest single wait inside this kernel.  The sharded form may be told to wait longer for its peers;
    // every other wait then gets twice that, so that the wait for the peers is the one that gives up first.
    const unsigned long long limit_ns = SEED == kSeedPeers ? 2ull * shard->wait_ns : kWaitLimitNs;
    constexpr int S = kSlots;
    extern __shared__ __align__(128) unsigned char p_smem[];
    E* slots = reinterpret_cast<E*>(p_smem);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(p_smem + S * kSlotBytes);  // tile landed in the slot
    uint64_t* agg_bar = full_bar + S;                                           // phase A done, aggregate known
    uint64_t* pre_bar = agg_bar + S;                                            // exclusive prefix known
    uint64_t* empty_bar = pre_bar + S;                                          // phase B done, slot reusable
    u64* s_agg64 = reinterpret_cast<u64*>(empty_bar + S);       // the three value arrays are laid out for 8-byte elements
    u64* s_excl64 = s_agg64 + S;
    u64* s_warp_total64 = s_excl64 + S;                          // [2][8]
    E* s_agg = reinterpret_cast<E*>(s_agg64);
    E* s_excl = reinterpret_cast<E*>(s_excl64);
    E* s_warp_total = reinterpret_cast<E*>(s_warp_total64);
    uint32_t* s_tile = reinterpret_cast<uint32_t*>(s_warp_total64 + 16);
    volatile uint32_t* abort_flag = s_tile + S;
    volatile uint32_t* s_ctrl = s_tile + S + 1;      // [2]: outcome of thread 0's bounded wait, double-buffered
    volatile uint32_t* s_end_item = s_tile + S + 3;  // ring item that carried the end-of-work mark

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const uint32_t tiles = static_cast<uint32_t>((static_cast<unsigned long long>(n) + TILE - 1) / TILE);

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&agg_bar[s], 1);
            mbar_init(&pre_bar[s], 1);
            mbar_init(&empty_bar[s], kScanThreads / 32);
        }
        *abort_flag = 0;
        *s_end_item = 0xFFFFFFFFu;
        fence_barrier_init();
    }
    __syncthreads();

    if constexpr (SEED == kSeedPeers) {
        if (shard->phases & kPhaseReduce)
            reduce_and_publish(n, static_cast<const uint32_t*>(src_v), header, *shard, s_tile,
                               reinterpret_cast<volatile uint32_t*>(s_warp_total64));
        if (!(shard->phases & kPhaseScan)) return;
        __syncthreads();
    }

    if (warp == kScanThreads / 32) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            for (uint32_t i = 0;; ++i) {
                const int s = i % S;
                if (!mbar_wait_bounded(&empty_bar[s], ((i / S) & 1u) ^ 1u, abort_flag, limit_ns)) {
                    *abort_flag = 1;
                    atomicExch(header + 1, 1u);
                    raise_device_status(DEV_SCAN_LOOKBACK_TIMEOUT);
                    break;
                }
                // The ticket of the reference (generated/get_block_idx_from_global_counter.cu:1-13),
                // drawn only now that the tile has somewhere to go.
                const uint32_t t = atomicAdd(header, 1u);
                if (t >= tiles) {
                    s_tile[s] = kSentinel;
                    mbar_arrive(&full_bar[s]);
                    break;
                }
                s_tile[s] = t;
                const unsigned long long base = static_cast<unsigned long long>(t) * TILE;
                const unsigned long long left = n - base;
                const uint32_t cnt = left < TILE ? static_cast<uint32_t>(left) : TILE;
                const uint32_t bytes = (cnt * static_cast<uint32_t>(sizeof(E))) & ~15u;  // whole 16-byte vectors; a ragged end is read by its owner
                if (bytes) {
                    mbar_arrive_expect_tx(&full_bar[s], bytes);
                    bulk_load_tile(slots + s * TILE, src + base, bytes, &full_bar[s]);
                } else {
                    mbar_arrive(&full_bar[s]);
                }
            }
        }
        return;
    }

    if (warp > kScanThreads / 32) {
        // ------------------------------ look-back ------------------------------
        static_assert(kLookbackWarps >= 1 && kLookbackWarps <= kSlots, "one look-back warp per slot at most");
        if constexpr (SEED == kSeedPeers) {
            // An empty chunk has no tile 0 to do the waiting, but the protocol still needs this rank to have seen
            // every word of this epoch before it moves on to the next one.
            if (tiles == 0 && blockIdx.x == 0) {
                bool failed = false;
                (void)wait_peer_words(*shard, abort_flag, &failed);
                if (failed && lane == 0) {
                    atomicExch(header + 1, 1u);
                    raise_device_status(DEV_SCAN_LOOKBACK_TIMEOUT);
                }
            }
        }
        for (uint32_t k = static_cast<uint32_t>(warp - kScanThreads / 32 - 1);; k += kLookbackWarps) {
            const int s = k % S;
            const bool ready = mbar_wait_bounded(&agg_bar[s], (k / S) & 1u, abort_flag, limit_ns);
            if (!__all_sync(0xffffffffu, ready)) {
                if (lane == 0) {
                    *abort_flag = 1;
                    atomicExch(header + 1, 1u);
                    raise_device_status(DEV_SCAN_LOOKBACK_TIMEOUT);
                }
                break;
            }
            if (k >= *s_end_item) break;   // the work ended before this ring item
            const uint32_t t = s_tile[s];
            const E agg = s_agg[s];
            E exclusive = 0;
            bool failed = false;
            if (t == 0) {
                if constexpr (SEED == kSeedTotals) {
                    const uint32_t* totals = static_cast<const uint32_t*>(seed_src);
                    for (int r = 0; r < rank; ++r) exclusive += totals[r];
                } else if constexpr (SEED == kSeedPeers) {
                    exclusive = wait_peer_words(*shard, abort_flag, &failed);
                }
            } else {
                exclusive = lookback<F32, E>(t, desc, header + 1, limit_ns, &failed);
            }
            if (lane == 0) {
                if (failed) {
                    *abort_flag = 1;
                    atomicExch(header + 1, 1u);
                    raise_device_status(DEV_SCAN_LOOKBACK_TIMEOUT);
                }
                rec_publish<E>(desc + static_cast<size_t>(t) * kRecStride, kStatePrefix, eadd<F32, E>(exclusive, agg));  // as write_block_prefix.cu:8-10
                s_excl[s] = exclusive;
                mbar_arrive(&pre_bar[s]);
            }
            __syncwarp();
            if (failed) break;
        }
        return;
    }

    // ------------------------------ scan warps ------------------------------
    // Lane l of warp w owns the 16-byte vectors at tile-local elements
    // w * kVecs * CHUNK + q * CHUNK + l * EPV (q = 0..3), in phase A and again in phase B.
    const int vec0 = warp * (kVecs * CHUNK) + lane * EPV;
    uint32_t i = 0, j = 0;  // ring items taken through phase A / phase B so far
    bool drained = false;
    // Scheduling.  Phase A (which publishes the aggregate that every later tile waits for) runs as
    // soon as a slot has landed, however many tiles are parked; phase B runs when the oldest parked
    // tile's prefix is there.  Only thread 0 watches the two barriers, with a time limit; what it
    // decides reaches the other 255 scan threads through a named barrier, so that all of them always
    // take the same branch (a thread that gave up on its own would leave the others stuck at the
    // next barrier).  The decision word is double-buffered because thread 0 can be one barrier ahead.
    uint32_t decisions = 0;
    auto decide = [&]() -> uint32_t {   // 0 = give up, 1 = phase A, 2 = phase B, 3 = all done
        volatile uint32_t* c = s_ctrl + (decisions++ & 1u);
        if (tid == 0) {
            uint32_t what = 0;
            const bool can_a = !drained && i - j < static_cast<uint32_t>(S);
            const bool can_b = j < i;
            if (!can_a && !can_b) {
                what = 3;
            } else {
                const unsigned long long t0 = global_timer_ns();
                for (uint32_t spin = 0;; ++spin) {
                    if (can_a && mbar_try_wait(&full_bar[i % S], (i / S) & 1u)) { what = 1; break; }
                    if (can_b && mbar_try_wait(&pre_bar[j % S], (j / S) & 1u)) { what = 2; break; }
                    if ((spin & 63u) == 63u && (*abort_flag || global_timer_ns() - t0 > limit_ns)) break;
                }
                if (what == 0) {
                    *abort_flag = 1;
                    atomicExch(header + 1, 1u);
                    raise_device_status(DEV_SCAN_LOOKBACK_TIMEOUT);
                }
            }
            *c = what;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kScanThreads) : "memory");
        return *c;
    };
    // A 16-byte vector as EPV elements and back.
    auto unpack = [](const uint4& v, E (&e)[EPV]) {
        if constexpr (I64) {
            e[0] = static_cast<u64>(v.x) | (static_cast<u64>(v.y) << 32);
            e[1] = static_cast<u64>(v.z) | (static_cast<u64>(v.w) << 32);
        } else {
            e[0] = v.x; e[1] = v.y; e[2] = v.z; e[3] = v.w;
        }
    };
    auto pack = [](const E (&e)[EPV]) -> uint4 {
        if constexpr (I64)
            return make_uint4(static_cast<uint32_t>(e[0]), static_cast<uint32_t>(e[0] >> 32), static_cast<uint32_t>(e[1]),
                              static_cast<uint32_t>(e[1] >> 32));
        else
            return make_uint4(e[0], e[1], e[2], e[3]);
    };

    while (true) {
        const uint32_t what = decide();
        if (what == 0 || what == 3) break;
        if (what == 1) {
            // ---------------- phase A on ring item i ----------------
            const int s = i % S;
            (void)mbar_try_wait(&full_bar[s], (i / S) & 1u);   // this thread's own acquire of the completed phase
            const uint32_t t = s_tile[s];
            if (t == kSentinel) {
                drained = true;
                if (tid == 0) {
                    // Wake every look-back warp at its next ring item and tell it that the work ended here.
                    *s_end_item = i;
                    for (int m = 0; m < kLookbackWarps; ++m) mbar_arrive(&agg_bar[(i + m) % S]);
                }
                continue;
            }
            E* slot = slots + s * TILE;
            const unsigned long long base = static_cast<unsigned long long>(t) * TILE;
            const unsigned long long left = n - base;
            const uint32_t cnt = left < TILE ? static_cast<uint32_t>(left) : TILE;
            E v[kVecs][EPV];
#pragma unroll
            for (int q = 0; q < kVecs; ++q) {
                const uint32_t e = vec0 + q * CHUNK;
                if (e + EPV <= (cnt & ~static_cast<uint32_t>(EPV - 1))) {
                    unpack(*reinterpret_cast<const uint4*>(slot + e), v[q]);
                } else {  // the ragged end of the last tile: straight from global memory, zero beyond n
#pragma unroll
                    for (int k = 0; k < EPV; ++k) v[q][k] = (e + k < cnt) ? src[base + e + k] : E(0);
                }
            }
            // Inside each 16-byte group, then across the 32 lanes of each of the four chunks
            // (the work of scan_warps.cu / naive_scan_warp_ends.cu in the reference).
            E sum[kVecs], inc[kVecs];
#pragma unroll
            for (int q = 0; q < kVecs; ++q) {
#pragma unroll
                for (int k = 1; k < EPV; ++k) v[q][k] = eadd<F32, E>(v[q][k], v[q][k - 1]);
                sum[q] = v[q][EPV - 1];
                inc[q] = sum[q];
            }
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
#pragma unroll
                for (int q = 0; q < kVecs; ++q) {
                    const E up = __shfl_up_sync(0xffffffffu, inc[q], d);
                    if (lane >= d) inc[q] = eadd<F32, E>(inc[q], up);
                }
            }
            E chunk_off = 0, excl[kVecs];
#pragma unroll
            for (int q = 0; q < kVecs; ++q) {
                if constexpr (F32) {   // no subtraction in floating point: the lane below's inclusive value
                    const E below = __shfl_up_sync(0xffffffffu, inc[q], 1);
                    excl[q] = eadd<F32, E>(chunk_off, lane == 0 ? E(0) : below);
                } else {
                    excl[q] = chunk_off + inc[q] - sum[q];
                }
                chunk_off = eadd<F32, E>(chunk_off, __shfl_sync(0xffffffffu, inc[q], 31));
            }
            E* wt = s_warp_total + (i & 1u) * 8;
            if (lane == 0) wt[warp] = chunk_off;
            asm volatile("bar.sync 1, %0;" ::"n"(kScanThreads) : "memory");
            E warp_off = 0, aggregate = 0;
#pragma unroll
            for (int w = 0; w < kScanThreads / 32; ++w) {
                const E tot = wt[w];
                if (w < warp) warp_off = eadd<F32, E>(warp_off, tot);
                aggregate = eadd<F32, E>(aggregate, tot);
            }
            if (tid == 0) {
                if (t != 0) rec_publish<E>(desc + static_cast<size_t>(t) * kRecStride, kStateAggregate, aggregate);  // as write_block_aggregate.cu:8-10
                s_agg[s] = aggregate;
                mbar_arrive(&agg_bar[s]);
            }
            // Tile-local inclusive scan back into the slot; the same lane reads it again in phase B.
#pragma unroll
            for (int q = 0; q < kVecs; ++q) {
                const E a = eadd<F32, E>(warp_off, excl[q]);
                if constexpr (EXCL) {   // each element gets the sum of the ones before it
#pragma unroll
                    for (int k = EPV - 1; k > 0; --k) v[q][k] = eadd<F32, E>(v[q][k - 1], a);
                    v[q][0] = a;
                } else {
#pragma unroll
                    for (int k = 0; k < EPV; ++k) v[q][k] = eadd<F32, E>(v[q][k], a);
                }
                *reinterpret_cast<uint4*>(slot + vec0 + q * CHUNK) = pack(v[q]);
            }
            ++i;
        } else {
            // ---------------- phase B on ring item j (update_with_new_data_and_writeback.cu) ----------------
            const int s = j % S;
            (void)mbar_try_wait(&pre_bar[s], (j / S) & 1u);
            const uint32_t t = s_tile[s];
            const E add = s_excl[s];
            const E* slot = slots + s * TILE;
            const unsigned long long base = static_cast<unsigned long long>(t) * TILE;
            const unsigned long long left = n - base;
            const uint32_t cnt = left < TILE ? static_cast<uint32_t>(left) : TILE;
#pragma unroll
            for (int q = 0; q < kVecs; ++q) {
                const uint32_t e = vec0 + q * CHUNK;
                E v[EPV];
                unpack(*reinterpret_cast<const uint4*>(slot + e), v);
#pragma unroll
                for (int k = 0; k < EPV; ++k) v[k] = eadd<F32, E>(v[k], add);
                if (e + EPV <= cnt) {
                    __stcg(reinterpret_cast<uint4*>(x + base + e), pack(v));
                } else {
#pragma unroll
                    for (int k = 0; k < EPV; ++k)
                        if (e + k < cnt) x[base + e + k] = v[k];
                }
            }
            // The slot was written with ordinary stores; the next write comes from the bulk-copy engine.
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
            ++j;
        }
    }
}

}  // namespace

// Same parameter list as the reference entry point (generated/scan_kernel.cu:1):
// n elements, data in place, the ticket counter, the per-tile records.  Here the
// counter word is followed by an abort flag and a record is one 64-bit word.
constexpr int kCtasPerSm = static_cast<int>((227 * 1024) / (kSmemBytes + 1024));

__global__ void __launch_bounds__(kThreads, kCtasPerSm)
scan_kernel(uint32_t n, uint32_t* x, uint32_t* block_idx_counter, int* block_infos) {
    scan_body<kSeedNone>(n, x, x, block_idx_counter, reinterpret_cast<uint64_t*>(block_infos), nullptr, 0);
}

// fp32 flavour of the same kernel (the reference scans uint32 only): same pipeline, fp32 adds.  The
// grouping of the partial sums follows the look-back windows, which depend on timing, so results can
// differ from run to run in the last bits, as with any floating-point decoupled look-back scan.
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
scan_kernel_f32(uint32_t n, float* x, uint32_t* block_idx_counter, int* block_infos) {
    scan_body<kSeedNone, true>(n, reinterpret_cast<uint32_t*>(x), reinterpret_cast<uint32_t*>(x), block_idx_counter,
                               reinterpret_cast<uint64_t*>(block_infos), nullptr, 0);
}

// General flavour (no counterpart in the reference): separate input and output, inclusive or exclusive,
// uint32 or fp32 adds.  in == out is allowed.
template <bool F32, bool EXCL>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
scan_kernel_general(uint32_t n, const uint32_t* in, uint32_t* out, uint32_t* block_idx_counter, int* block_infos) {
    scan_body<kSeedNone, F32, EXCL>(n, in, out, block_idx_counter, reinterpret_cast<uint64_t*>(block_infos), nullptr, 0);
}

// 64-bit integer flavour (no counterpart in the reference, whose scan is uint32 only): the same pipeline on
// 2048-element tiles, a tile's record split over two 64-bit words.
template <bool EXCL>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
scan_kernel_i64(uint32_t n, const unsigned long long* in, unsigned long long* out, uint32_t* block_idx_counter,
                int* block_infos) {
    scan_body<kSeedNone, false, EXCL, true>(n, in, out, block_idx_counter, reinterpret_cast<uint64_t*>(block_infos), nullptr, 0);
}

// Sharded form: tile 0 starts from totals[0] + ... + totals[rank-1].
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
scan_kernel_seeded(uint32_t n, uint32_t* x, uint32_t* block_idx_counter, int* block_infos, const uint32_t* totals,
                   int rank) {
    scan_body<kSeedTotals>(n, x, x, block_idx_counter, reinterpret_cast<uint64_t*>(block_infos), totals, rank);
}

// Sharded form without a collective call, in one launch: (1) the chunk's total, stored as an {epoch, total}
// word into every rank's memory by whichever CTA finishes the last slice, (2) the scan, whose first tile
// waits for all ranks' words and starts from the sum of the lower ranks' totals.  Either phase can be
// switched off (the two-launch form, and the emulation of several ranks on one GPU, where a launch
// that waits for a later launch's word would never see it).
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
scan_kernel_sharded(uint32_t n, uint32_t* x, uint32_t* block_idx_counter, int* block_infos, const ShardArgs shard) {
    scan_body<kSeedPeers>(n, x, x, block_idx_counter, reinterpret_cast<uint64_t*>(block_infos), nullptr, shard.rank, &shard);
}

// Stores this rank's {epoch, total} word into every rank's slot array (its own included) with one
// 64-bit system-scope store each: lane p writes to rank p's memory over NVLink.
__global__ void publish_total_kernel(const uint32_t* total, uint64_t* const* peer_slots, int world, int rank,
                                     uint32_t epoch) {
    const int p = threadIdx.x;
    if (p < world) {
        const uint64_t w = static_cast<uint64_t>(epoch) | (static_cast<uint64_t>(*total) << 32);
        uint64_t* dst = peer_slots[p] + (epoch & 1u) * world + rank;
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(w) : "memory");
    }
}

__global__ void __launch_bounds__(256) reduce_u32_kernel(size_t n, const uint32_t* x, uint32_t* total) {
    __shared__ uint32_t s_part[8];
    uint32_t acc = 0;
    const size_t n4 = n / 4;
    const uint4* x4 = reinterpret_cast<const uint4*>(x);
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    // The array is walked from its end to its start, so that what is still in L2 when the scan pass
    // begins is the part the scan reads first.  Four independent 16-byte loads in flight per thread.
    const uint4* top = x4 + (n4 - 1);
    for (; i + 3 * stride < n4; i += 4 * stride) {
        const uint4 a = __ldcg(top - i), b = __ldcg(top - (i + stride)), c = __ldcg(top - (i + 2 * stride)),
                    d = __ldcg(top - (i + 3 * stride));
        acc += (a.x + a.y) + (a.z + a.w) + (b.x + b.y) + (b.z + b.w) + (c.x + c.y) + (c.z + c.w) + (d.x + d.y) +
               (d.z + d.w);
    }
    for (; i < n4; i += stride) {
        const uint4 a = __ldcg(top - i);
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

// Tiles of n elements of elem_bytes (4 or 8) each: a tile is always 16 KB.
size_t scan_tiles(size_t n, size_t elem_bytes = 4) {
    const size_t per_tile = kSlotBytes / elem_bytes;
    return (n + per_tile - 1) / per_tile;
}

// Resident CTAs of the persistent kernel on the current device (SMs x CTAs per SM), found
// once per device; also raises the kernels' dynamic shared-memory limit.
int persistent_grid(unsigned* out) {
    static unsigned cached[64] = {};
    static std::mutex mu;   // entry points may be called from several host threads
    std::lock_guard<std::mutex> lk(mu);
    int dev = 0;
    PRISM_CUDA_TRY(cudaGetDevice(&dev));
    const bool cacheable = dev >= 0 && dev < 64;
    if (cacheable && cached[dev]) {
        *out = cached[dev];
        return PRISM_B200_OK;
    }
    int sms = 0, per_sm = 0;
    PRISM_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    PRISM_CUDA_TRY(cudaFuncSetAttribute(scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(kSmemBytes)));
    PRISM_CUDA_TRY(cudaFuncSetAttribute(scan_kernel_seeded, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(kSmemBytes)));
    PRISM_CUDA_TRY(cudaFuncSetAttribute(scan_kernel_f32, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(kSmemBytes)));
    PRISM_CUDA_TRY(cudaFuncSetAttribute(scan_kernel_general<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(kSmemBytes)));
    PRISM_CUDA_TRY(cudaFuncSetAttribute(scan_kernel_general<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(kSmemBytes)));
    PRISM_CUDA_TRY(cudaFuncSetAttribute(scan_kernel_general<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(kSmemBytes)));
    PRISM_CUDA_TRY(cudaFuncSetAttribute(scan_kernel_general<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(kSmemBytes)));
    PRISM_CUDA_TRY(cudaFuncSetAttribute(scan_kernel_i64<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(kSmemBytes)));
    PRISM_CUDA_TRY(cudaFuncSetAttribute(scan_kernel_i64<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(kSmemBytes)));
    PRISM_CUDA_TRY(cudaFuncSetAttribute(scan_kernel_sharded, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(kSmemBytes)));
    PRISM_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, scan_kernel, kThreads, kSmemBytes));
    if (per_sm < 1 || sms < 1) return set_error(PRISM_B200_ERR_CUDA, "scan: the kernel does not fit on an SM");
    *out = static_cast<unsigned>(sms * per_sm);
    if (cacheable) cached[dev] = *out;
    return PRISM_B200_OK;
}

// Re-arms the scratch (ticket, abort flag, every record: one memset where the reference
// issues two, evals/4090_scan/main.cu:81-82) and launches the kernel.
int scan_enqueue(size_t n, uint32_t* x, void* scratch, const void* seed_src, int rank, int seed_mode,
                 cudaStream_t stream, const ShardArgs* shard = nullptr) {
    const uint32_t tiles = static_cast<uint32_t>(scan_tiles(n));
    uint32_t* header = static_cast<uint32_t*>(scratch);
    uint64_t* desc = reinterpret_cast<uint64_t*>(static_cast<char*>(scratch) + kHeaderBytes);
    unsigned grid = 0;
    if (int rc = persistent_grid(&grid)) return rc;
    if (grid > tiles) grid = tiles > 0 ? tiles : 1;   // tiles == 0 only in the sharded form (an empty chunk)
    PRISM_CUDA_TRY(cudaMemsetAsync(scratch, 0, kHeaderBytes + static_cast<size_t>(tiles) * kRecStride * sizeof(uint64_t), stream));
    if (seed_mode == kSeedPeers)
        scan_kernel_sharded<<<grid, kThreads, kSmemBytes, stream>>>(static_cast<uint32_t>(n), x, header,
                                                                    reinterpret_cast<int*>(desc), *shard);
    else if (seed_mode == kSeedTotals)
        scan_kernel_seeded<<<grid, kThreads, kSmemBytes, stream>>>(static_cast<uint32_t>(n), x, header,
                                                                   reinterpret_cast<int*>(desc),
                                                                   static_cast<const uint32_t*>(seed_src), rank);
    else if (seed_mode == kSeedNoneF32)
        scan_kernel_f32<<<grid, kThreads, kSmemBytes, stream>>>(static_cast<uint32_t>(n), reinterpret_cast<float*>(x), header,
                                                                reinterpret_cast<int*>(desc));
    else
        scan_kernel<<<grid, kThreads, kSmemBytes, stream>>>(static_cast<uint32_t>(n), x, header,
                                                            reinterpret_cast<int*>(desc));
    PRISM_CUDA_TRY(cudaGetLastError());
    count_launch();
    return PRISM_B200_OK;
}

int scan_launch(size_t n, uint32_t* x, void* workspace, const void* seed_src, int rank, int seed_mode,
                cudaStream_t stream) {
    if (n == 0) return PRISM_B200_OK;
    if (!x || !workspace) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "scan: null pointer");
    if (n >= (1ull << 32)) return set_error(PRISM_B200_ERR_TOO_LARGE, "scan: n=%zu must be below 2^32", n);
    if (reinterpret_cast<uintptr_t>(x) & 15u) return set_error(PRISM_B200_ERR_MISALIGNED, "scan: x not 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(workspace) & 15u)
        return set_error(PRISM_B200_ERR_MISALIGNED, "scan: workspace not 16-byte aligned");
    if (seed_mode == kSeedTotals && (rank < 0 || (rank > 0 && !seed_src)))
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "scan_seeded: bad rank/totals");
    if (int rc = bind_status_word()) return rc;
    return scan_enqueue(n, x, workspace, seed_src, rank, seed_mode, stream);
}

// The sharded form.  Unlike the others it runs for n == 0 too: an empty chunk still has to publish its
// word and to wait for the others'.
int scan_sharded_launch(size_t n, uint32_t* x, void* workspace, const uint64_t* slots, uint64_t* const* peer_slots,
                        int rank, int world, uint32_t epoch, int phases, unsigned long long wait_limit_ns,
                        cudaStream_t stream) {
    if (phases < 1 || phases > 3) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "scan_sharded: phases must be 1, 2 or 3");
    // rank == world with the scan phase alone: a piece that lies behind every rank's chunk (it publishes nothing and
    // is seeded with the sum of all the ranks' totals).
    const bool behind_all = rank == world && phases == kPhaseScan;
    if (world < 1 || world > 32 || rank < 0 || (rank >= world && !behind_all) || epoch == 0)
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT,
                         "scan_sharded: need 1 <= world <= 32, a rank below world (or equal to it, scan phase only) and a "
                         "non-zero epoch");
    if (((phases & kPhaseReduce) && !peer_slots) || ((phases & kPhaseScan) && !slots) || !workspace || (n && !x))
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "scan_sharded: null pointer");
    if (n >= (1ull << 32)) return set_error(PRISM_B200_ERR_TOO_LARGE, "scan_sharded: n=%zu must be below 2^32", n);
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(workspace)) & 15u)
        return set_error(PRISM_B200_ERR_MISALIGNED, "scan_sharded: x and workspace must be 16-byte aligned");
    if (wait_limit_ns == 0) wait_limit_ns = kWaitLimitNs;
    if (wait_limit_ns > 600ull * kWaitLimitNs)
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "scan_sharded: wait limit above 600 s");
    if (int rc = bind_status_word()) return rc;
    const ShardArgs shard{slots, peer_slots, rank, world, epoch, static_cast<uint32_t>(phases), wait_limit_ns};
    return scan_enqueue(n, x, workspace, nullptr, rank, kSeedPeers, stream, &shard);
}

// The general flavour: same re-arming and grid as scan_enqueue.
int scan_general_launch(size_t n, const void* in, void* out, void* workspace, int flags, cudaStream_t stream) {
    if (flags & ~(PRISM_B200_SCAN_EXCLUSIVE | PRISM_B200_SCAN_F32 | PRISM_B200_SCAN_I64))
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "scan_general: unknown flag bits 0x%x", flags);
    if ((flags & PRISM_B200_SCAN_F32) && (flags & PRISM_B200_SCAN_I64))
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "scan_general: F32 and I64 exclude each other");
    if (n == 0) return PRISM_B200_OK;
    if (!in || !out || !workspace) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "scan_general: null pointer");
    if (n >= (1ull << 32)) return set_error(PRISM_B200_ERR_TOO_LARGE, "scan_general: n=%zu must be below 2^32", n);
    if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(workspace)) & 15u)
        return set_error(PRISM_B200_ERR_MISALIGNED, "scan_general: in, out and workspace must be 16-byte aligned");
    const size_t elem = (flags & PRISM_B200_SCAN_I64) ? 8 : 4;
    if (in != out) {
        const uintptr_t a = reinterpret_cast<uintptr_t>(in), b = reinterpret_cast<uintptr_t>(out);
        if (a < b + n * elem && b < a + n * elem)
            return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "scan_general: in and out overlap without being equal");
    }
    if (int rc = bind_status_word()) return rc;
    const uint32_t tiles = static_cast<uint32_t>(scan_tiles(n, elem));
    uint32_t* header = static_cast<uint32_t*>(workspace);
    int* desc = reinterpret_cast<int*>(static_cast<char*>(workspace) + kHeaderBytes);
    unsigned grid = 0;
    if (int rc = persistent_grid(&grid)) return rc;
    if (grid > tiles) grid = tiles;
    PRISM_CUDA_TRY(cudaMemsetAsync(workspace, 0, kHeaderBytes + static_cast<size_t>(tiles) * kRecStride * sizeof(uint64_t), stream));
    const uint32_t n32 = static_cast<uint32_t>(n);
    const uint32_t* in32 = static_cast<const uint32_t*>(in);
    uint32_t* out32 = static_cast<uint32_t*>(out);
    const unsigned long long* in64 = static_cast<const unsigned long long*>(in);
    unsigned long long* out64 = static_cast<unsigned long long*>(out);
    switch (flags) {
    case 0: scan_kernel_general<false, false><<<grid, kThreads, kSmemBytes, stream>>>(n32, in32, out32, header, desc); break;
    case PRISM_B200_SCAN_EXCLUSIVE: scan_kernel_general<false, true><<<grid, kThreads, kSmemBytes, stream>>>(n32, in32, out32, header, desc); break;
    case PRISM_B200_SCAN_F32: scan_kernel_general<true, false><<<grid, kThreads, kSmemBytes, stream>>>(n32, in32, out32, header, desc); break;
    case PRISM_B200_SCAN_F32 | PRISM_B200_SCAN_EXCLUSIVE: scan_kernel_general<true, true><<<grid, kThreads, kSmemBytes, stream>>>(n32, in32, out32, header, desc); break;
    case PRISM_B200_SCAN_I64: scan_kernel_i64<false><<<grid, kThreads, kSmemBytes, stream>>>(n32, in64, out64, header, desc); break;
    default: scan_kernel_i64<true><<<grid, kThreads, kSmemBytes, stream>>>(n32, in64, out64, header, desc); break;
    }
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
constexpr size_t kStaticScratchBytes = kHeaderBytes + (kStaticMaxN / kTile) * kRecStride * sizeof(uint64_t);  // 2,097,280 B
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
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
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
    // The array still holds the previous call's ticket, abort flag and records; scan_enqueue clears
    // what this call will use.  It does not set up the pinned status word (that would allocate).
    return scan_enqueue(n, x, scratch, nullptr, 0, kSeedNone, static_cast<cudaStream_t>(stream));
}


extern "C" int prism_b200_scan_workspace_size(size_t n, size_t* bytes) {
    if (!bytes) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "scan_workspace_size: null bytes");
    if (n >= (1ull << 32)) return set_error(PRISM_B200_ERR_TOO_LARGE, "scan: n=%zu must be below 2^32", n);
    *bytes = kHeaderBytes + scan_tiles(n) * kRecStride * sizeof(uint64_t);
    return PRISM_B200_OK;
}

extern "C" int prism_b200_scan(size_t n, uint32_t* x, void* workspace, void* stream) {
    return scan_launch(n, x, workspace, nullptr, 0, kSeedNone, static_cast<cudaStream_t>(stream));
}

extern "C" int prism_b200_scan_f32(size_t n, float* x, void* workspace, void* stream) {
    return scan_launch(n, reinterpret_cast<uint32_t*>(x), workspace, nullptr, 0, kSeedNoneF32,
                       static_cast<cudaStream_t>(stream));
}

extern "C" int prism_b200_scan_general(size_t n, const void* in, void* out, void* workspace, int flags, void* stream) {
    return scan_general_launch(n, in, out, workspace, flags, static_cast<cudaStream_t>(stream));
}

extern "C" int prism_b200_scan_general_workspace_size(size_t n, int flags, size_t* bytes) {
    if (!bytes) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "scan_general_workspace_size: null bytes");
    if (n >= (1ull << 32)) return set_error(PRISM_B200_ERR_TOO_LARGE, "scan: n=%zu must be below 2^32", n);
    *bytes = kHeaderBytes + scan_tiles(n, (flags & PRISM_B200_SCAN_I64) ? 8 : 4) * kRecStride * sizeof(uint64_t);
    return PRISM_B200_OK;
}

extern "C" int prism_b200_scan_seeded(size_t n, uint32_t* x, void* workspace, const uint32_t* totals, int rank,
                                      void* stream) {
    return scan_launch(n, x, workspace, totals, rank, kSeedTotals, static_cast<cudaStream_t>(stream));
}

extern "C" int prism_b200_scan_publish_total(const uint32_t* total, uint64_t* const* peer_slots, int world, int rank,
                                             uint32_t epoch, void* stream) {
    if (!total || !peer_slots || world < 1 || world > 32 || rank < 0 || rank >= world || epoch == 0)
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "scan_publish_total: bad argument");
    publish_total_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(total, peer_slots, world, rank, epoch);
    PRISM_CUDA_TRY(cudaGetLastError());
    count_launch();
    return PRISM_B200_OK;
}

extern "C" int prism_b200_scan_seeded_peers(size_t n, uint32_t* x, void* workspace, const uint64_t* slots, int rank,
                                            int world, uint32_t epoch, void* stream) {
    return scan_sharded_launch(n, x, workspace, slots, nullptr, rank, world, epoch, kPhaseScan, 0,
                               static_cast<cudaStream_t>(stream));
}

extern "C" int prism_b200_scan_sharded(size_t n, uint32_t* x, void* workspace, const uint64_t* slots,
                                       uint64_t* const* peer_slots, int rank, int world, uint32_t epoch, int phases,
                                       unsigned long long wait_limit_ns, void* stream) {
    return scan_sharded_launch(n, x, workspace, slots, peer_slots, rank, world, epoch, phases, wait_limit_ns,
                               static_cast<cudaStream_t>(stream));
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
