// bf16 GEMM for B200: C = A * B^T with fp32 accumulation on the 5th-generation
// tensor cores (tcgen05.mma, accumulators in tensor memory), operands staged by
// TMA, persistent CTAs.
//
// What it stands in for: `cutlass_my_h100_match_no_tail`
// (generated/cutlass_my_h100_match_no_tail.cu:1-370), a Hopper kernel built on
// wgmma/setmaxnreg that does not assemble for sm_100a, and its launcher
// `runmyh100` (evals/h100_bench/utils.cuh:504-533).  Same data contract:
//   A  M x K  bf16, K contiguous         B  N x K  bf16, K contiguous
//   C  M x N  bf16, COLUMN-major: C[n * M + m]   (cutlass_my_h100_match_no_tail.cu:313,347-354)
// and the same kernel parameter list (M, N, K, C, tensorMapA, tensorMapB).
//
// Design.
//   * Column-major C is row-major C^T = B * A^T, so the kernel computes C^T: the
//     rows of B index the 128 TMEM lanes of an accumulator and the rows of A index
//     its columns.  A thread that reads one TMEM lane then holds consecutive m of a
//     single n, which are consecutive in memory, so the epilogue writes 16-byte
//     vectors straight from registers with no transpose.
//   * CTA tile: 128 (n) x BLOCK_Q (m, 256 or 128) x 64 (k).  One tcgen05.mma covers
//     128 x BLOCK_Q x 16; four of them consume a stage.  Operands sit in shared
//     memory in the 128-byte-swizzled K-major layout that TMA writes and the MMA
//     descriptors name (8-row groups 1024 B apart).
//   * Warp roles: warp 0 issues TMA loads, warp 1 owns tensor memory and issues the
//     MMAs, warps 2-5 drain accumulators (each warp can reach one 32-lane quarter
//     of tensor memory, picked by warp index mod 4).
//   * Two accumulators (2 x BLOCK_Q columns of the 512) alternate, so the epilogue
//     of one tile overlaps the main loop of the next.
//   * Four mbarrier rings: smem full/empty per stage, accumulator full/empty.
//     tcgen05.commit makes the MMA completion arrive on a barrier.  Every wait is
//     bounded; a wait that runs out raises DEV_GEMM_PIPE_TIMEOUT, all roles
//     unwind, tensor memory is freed and the kernel returns.
//   * Tiles are dealt round-robin to the resident CTAs in an order that walks 8
//     m-tiles for each n-tile, so a wave of CTAs shares operand rows in L2.
#include "common.cuh"

#include <cuda.h>
#include <cuda_bf16.h>

#include <mutex>
#include <unordered_map>

namespace prism_b200 {

namespace g16 {
constexpr int BLOCK_P = 128;     // rows of B (n) per tile -> TMEM lanes
constexpr int BLOCK_K = 64;      // 64 bf16 = 128 bytes = one swizzle span
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int EPI_WARPS = 4;
constexpr int GROUP_M = 8;       // m-tiles walked per n-tile
constexpr int TMEM_COLS = 512;

template <int BLOCK_Q>
struct Cfg {
    static constexpr int STAGES = BLOCK_Q == 256 ? 4 : 6;
    static constexpr uint32_t P_BYTES = BLOCK_P * BLOCK_K * 2;
    static constexpr uint32_t Q_BYTES = BLOCK_Q * BLOCK_K * 2;
    static constexpr uint32_t STAGE_BYTES = P_BYTES + Q_BYTES;
    // 1024 B of slack to align the ring, then barriers and the TMEM slot.
    static constexpr size_t SMEM_BYTES = 1024 + static_cast<size_t>(STAGES) * STAGE_BYTES + (2 * STAGES + 4) * 8 + 16;
};

// Instruction descriptor for kind::f16: D = fp32, A = B = bf16, both K-major,
// N at bits 17-22 (N >> 3), M at bits 24-28 (M >> 4).
__host__ __device__ constexpr uint32_t instr_desc(int umma_m, int umma_n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(umma_n >> 3) << 17) |
           (static_cast<uint32_t>(umma_m >> 4) << 24);
}
}  // namespace g16

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 B
// apart (stride byte offset), descriptor version 1 (Blackwell).
__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;             // leading byte offset (unused with swizzle)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;     // stride byte offset
    d |= static_cast<uint64_t>(1) << 46;             // version
    d |= static_cast<uint64_t>(2) << 61;             // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrives on `bar` once every tcgen05.mma issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld_32cols(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(uint32_t lo_f32_bits, uint32_t hi_f32_bits) {
    const __nv_bfloat162 v = __float22bfloat162_rn(make_float2(__uint_as_float(lo_f32_bits), __uint_as_float(hi_f32_bits)));
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Tile t -> (n-tile, m-tile): GROUP_M m-tiles are walked for each n-tile before n advances.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn,
                                            int group_m = g16::GROUP_M) {
    const int per_group = group_m * tiles_n;
    const int group = t / per_group;
    const int first_m = group * group_m;
    const int rows = min(group_m, tiles_m - first_m);
    const int in = t - group * per_group;
    tm = first_m + in % rows;
    tn = in / rows;
}

// alpha * acc + beta * c for eight bf16 values of C held in a uint4, packed back to bf16.
__device__ __forceinline__ uint4 axpby8(const uint32_t* acc_bits, uint4 c, float alpha, float beta) {
    const uint32_t cw[4] = {c.x, c.y, c.z, c.w};
    uint32_t ow[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // beta == 0 means "Cin does not enter", whatever it holds (NaN included), as in BLAS
        const float c_lo = beta != 0.f ? beta * __uint_as_float(cw[i] << 16) : 0.f;
        const float c_hi = beta != 0.f ? beta * __uint_as_float(cw[i] & 0xFFFF0000u) : 0.f;
        const float lo = fmaf(alpha, __uint_as_float(acc_bits[2 * i]), c_lo);
        const float hi = fmaf(alpha, __uint_as_float(acc_bits[2 * i + 1]), c_hi);
        ow[i] = pack_bf16(__float_as_uint(lo), __float_as_uint(hi));
    }
    return make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

// AXPBY: the epilogue stores alpha * (A * B^T) + beta * Cin instead of A * B^T (Cin in C's layout; Cin == C allowed).
template <int BLOCK_Q, bool AXPBY>
__device__ __forceinline__ void single_cta_body(int M, int N, int K, __nv_bfloat16* C, const CUtensorMap* mapA,
                                                const CUtensorMap* mapB, float alpha, float beta,
                                                const __nv_bfloat16* Cin) {
    const CUtensorMap& tensorMapA = *mapA;
    const CUtensorMap& tensorMapB = *mapB;
    using namespace g16;
    using C_ = Cfg<BLOCK_Q>;
    constexpr int STAGES = C_::STAGES;
    constexpr uint32_t IDESC = instr_desc(BLOCK_P, BLOCK_Q);

    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    unsigned char* ring = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);  // 1024-byte aligned
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(ring + STAGES * C_::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full_bar = empty_bar + STAGES;   // [2]
    uint64_t* acc_empty_bar = acc_full_bar + 2;    // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* never_flag = tmem_slot + 2;  // stays 0: lets the unwind path wait although abort is set

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_m = M / BLOCK_Q;
    const int tiles_n = N / BLOCK_P;
    const int total_tiles = tiles_m * tiles_n;
    const int k_blocks = K / BLOCK_K;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full_bar[a], 1);
            mbar_init(&acc_empty_bar[a], EPI_WARPS);
        }
        *abort_flag = 0;
        *never_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(static_cast<uint32_t>(TMEM_COLS))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    bool timed_out = false;

    if (warp == 0) {
        // ------------------------- TMA producer -------------------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tensorMapA)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tensorMapB)) : "memory");
            int stage = 0;
            uint32_t phase = 0;
            int armed = 0;  // stages armed and not known to be consumed (for the unwind path)
            for (int t = blockIdx.x; t < total_tiles && !timed_out; t += gridDim.x) {
                int tm, tn;
                tile_coords(t, tiles_m, tiles_n, tm, tn);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait_bounded_sleepy(&empty_bar[stage], phase ^ 1u, abort_flag, 40)) {
                        timed_out = true;
                        break;
                    }
                    unsigned char* p_dst = ring + stage * C_::STAGE_BYTES;
                    unsigned char* q_dst = p_dst + C_::P_BYTES;
                    mbar_arrive_expect_tx(&full_bar[stage], C_::STAGE_BYTES);
                    tma_load_2d(p_dst, &tensorMapB, kb * BLOCK_K, tn * BLOCK_P, &full_bar[stage]);
                    tma_load_2d(q_dst, &tensorMapA, kb * BLOCK_K, tm * BLOCK_Q, &full_bar[stage]);
                    armed = armed < STAGES ? armed + 1 : STAGES;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (timed_out || *abort_flag) {
                // Unwind: let loads already in flight land before shared memory is released.
                int s = stage;
                uint32_t ph = phase;
                for (int i = 0; i < armed; ++i) {
                    if (--s < 0) {
                        s = STAGES - 1;
                        ph ^= 1u;
                    }
                    mbar_wait_bounded(&full_bar[s], ph, never_flag, 2000000ull);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------- MMA issuer -------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            for (int t = blockIdx.x; t < total_tiles && !timed_out; t += gridDim.x) {
                if (!mbar_wait_bounded(&acc_empty_bar[acc], acc_phase ^ 1u, abort_flag)) {
                    timed_out = true;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BLOCK_Q);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) {
                        timed_out = true;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t p_addr = smem_u32(ring + stage * C_::STAGE_BYTES);
                    const uint64_t p_desc = smem_desc_k_sw128(p_addr);
                    const uint64_t q_desc = smem_desc_k_sw128(p_addr + C_::P_BYTES);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        // 16 bf16 = 32 bytes further along K inside the swizzle span: +2 in the address field.
                        umma_bf16(d_tmem, p_desc + 2u * k, q_desc + 2u * k, IDESC, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[stage]);  // stage is free once these MMAs have read it
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (timed_out) break;
                umma_commit(&acc_full_bar[acc]);  // accumulator complete
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ------------------------- epilogue warps -------------------------
        const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 are reachable from this warp
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
            int tm, tn;
            tile_coords(t, tiles_m, tiles_n, tm, tn);
            // Warp-uniform outcome: the TMEM loads below need the whole warp converged.
            // One lane polls, with sleeps in between (the wait lasts most of a tile's main loop);
            // the other 31 lanes block at the vote.
            const bool ready = lane != 0 || mbar_wait_bounded_sleepy(&acc_full_bar[acc], acc_phase, abort_flag, 200);
            if (!__all_sync(0xffffffffu, ready)) {
                timed_out = true;
                break;
            }
            tc_fence_after();
            const size_t n = static_cast<size_t>(tn) * BLOCK_P + quarter * 32 + lane;
            const size_t c_off = n * static_cast<size_t>(M) + static_cast<size_t>(tm) * BLOCK_Q;
            __nv_bfloat16* c_row = C + c_off;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(acc * BLOCK_Q);
#pragma unroll 2
            for (int c = 0; c < BLOCK_Q; c += 32) {
                uint32_t r[32];
                tmem_ld_32cols(t_row + c, r);
                tmem_ld_wait();
                uint4* dst = reinterpret_cast<uint4*>(c_row + c);
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    uint4 o;
                    if constexpr (AXPBY) {
                        o = axpby8(&r[8 * v], reinterpret_cast<const uint4*>(Cin + c_off + c)[v], alpha, beta);
                    } else {
                        o.x = pack_bf16(r[8 * v + 0], r[8 * v + 1]);
                        o.y = pack_bf16(r[8 * v + 2], r[8 * v + 3]);
                        o.z = pack_bf16(r[8 * v + 4], r[8 * v + 5]);
                        o.w = pack_bf16(r[8 * v + 6], r[8 * v + 7]);
                    }
                    dst[v] = o;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty_bar[acc]);
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
    }

    if (timed_out) {
        *abort_flag = 1;
        raise_device_status(DEV_GEMM_PIPE_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(static_cast<uint32_t>(TMEM_COLS))
                     : "memory");
    }
}

template <int BLOCK_Q>
__global__ void __launch_bounds__(g16::THREADS, 1)
cutlass_my_h100_match_no_tail(int M, int N, int K, __nv_bfloat16* C, const __grid_constant__ CUtensorMap tensorMapA,
                              const __grid_constant__ CUtensorMap tensorMapB) {
    single_cta_body<BLOCK_Q, false>(M, N, K, C, &tensorMapA, &tensorMapB, 1.f, 0.f, nullptr);
}

// D = alpha * A * B^T + beta * Cin (no counterpart in the reference, whose kernel has no scaling epilogue).
template <int BLOCK_Q>
__global__ void __launch_bounds__(g16::THREADS, 1)
cutlass_my_h100_match_no_tail_axpby(int M, int N, int K, __nv_bfloat16* D, const __grid_constant__ CUtensorMap tensorMapA,
                                    const __grid_constant__ CUtensorMap tensorMapB, float alpha, float beta,
                                    const __nv_bfloat16* Cin) {
    single_cta_body<BLOCK_Q, true>(M, N, K, D, &tensorMapA, &tensorMapB, alpha, beta, Cin);
}

// ============================================================================
// Two-CTA form: a cluster of two CTAs on neighbouring SMs computes one 256 (n) x
// 256 (m) tile with tcgen05.mma.cta_group::2.  Each CTA loads its own 128 rows of
// both operands (32 KB per stage instead of 48 KB, six stages instead of four) and
// holds the accumulator rows of its own 128 n; the tensor cores of each SM read the
// other SM's half of the m-side operand through the pair, so every operand byte is
// staged once per pair instead of once per CTA.
//   * CTA 0 (the leader) issues every MMA.  The TMA loads of both CTAs complete on
//     the LEADER's "full" barrier (the .cta_group::2 form of the load allows the
//     barrier to live in the other CTA); the leader expects both CTAs' bytes.
//   * After the MMAs of a stage the leader commits twice: to its own "empty"
//     barrier and, through its cluster address, to the other CTA's.  The same for
//     "accumulator full".  No multicast qualifier is used anywhere.
//   * The epilogue warps of both CTAs arrive on the leader's "accumulator empty"
//     barrier (count 8).
//   * The two CTAs synchronise as a cluster after barrier set-up and before tensor
//     memory is released, so neither can touch a barrier or operand of a CTA that
//     is not there yet or has already left.
// ============================================================================
namespace g16 {
struct PairCfg {
    static constexpr int EPI_WARPS = 4;
    static constexpr int BLOCK = 256;      // tile edge of the pair, both in n and in m
    static constexpr int HALF = 128;       // rows of either operand staged by one CTA
    static constexpr int STAGES = 6;
    static constexpr uint32_t HALF_BYTES = HALF * BLOCK_K * 2;
    static constexpr uint32_t STAGE_BYTES = 2 * HALF_BYTES;  // per CTA
    static constexpr uint32_t BAR_BYTES = 256;                // barriers, TMEM slot, flags
    static constexpr uint32_t EPI_WARP_BYTES = 32 * 128;      // 32 rows x 64 bf16 per epilogue warp
    static constexpr size_t SMEM_BYTES =
        1024 + static_cast<size_t>(STAGES) * STAGE_BYTES + BAR_BYTES + EPI_WARPS * EPI_WARP_BYTES;
};
}  // namespace g16

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of a shared-memory object of CTA `rank` of this cluster, in the shared::cluster window.
__device__ __forceinline__ uint32_t cluster_addr(const void* smem_ptr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(smem_ptr)), "r"(rank));
    return out;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar_addr) : "memory");
}
// TMA load whose completion is counted on a barrier that may live in the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(cluster_bar)
        : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar_addr)
                 : "memory");
}

// Unwind path of the two-CTA kernels' producers: loads already issued must land before the CTA gives
// its shared memory back.  All loads of a pair complete on the LEADER's "full" barriers, so the
// leader waits for the armed ones (never_flag stays 0, so the wait is not cut short by the abort
// flag); the other CTA cannot watch those barriers and instead lets the longest a load can take
// pass.  Both are bounded.
__device__ __forceinline__ void drain_pair_loads(uint64_t* full_bar, int stage, uint32_t phase, int armed, int stages,
                                                 bool leader, volatile uint32_t* never_flag) {
    if (leader) {
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < armed; ++i) {
            if (--s < 0) {
                s = stages - 1;
                ph ^= 1u;
            }
            mbar_wait_bounded(&full_bar[s], ph, never_flag, 2000000ull);
        }
    } else if (armed > 0) {
        const unsigned long long t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
}

template <int GROUP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(g16::THREADS, 1)
cutlass_my_h100_match_no_tail_pair(int M, int N, int K, __nv_bfloat16* C, const __grid_constant__ CUtensorMap tensorMapA,
                                   const __grid_constant__ CUtensorMap tensorMapB) {
    using namespace g16;
    using P_ = PairCfg;
    constexpr int STAGES = P_::STAGES;
    constexpr uint32_t IDESC = instr_desc(P_::BLOCK, P_::BLOCK);  // M = 256 across the pair, N = 256

    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    unsigned char* ring = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);  // same offset in both CTAs
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(ring + STAGES * P_::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full_bar = empty_bar + STAGES;   // [2]
    uint64_t* acc_empty_bar = acc_full_bar + 2;    // [2], only the leader's are used
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* never_flag = tmem_slot + 2;
    unsigned char* epi_smem = ring + STAGES * P_::STAGE_BYTES + P_::BAR_BYTES;   // 128-byte aligned

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1;
    const int pairs = gridDim.x >> 1;
    const int tiles_m = M / P_::BLOCK;
    const int tiles_n = N / P_::BLOCK;
    const int total_tiles = tiles_m * tiles_n;
    const int k_blocks = K / BLOCK_K;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full_bar[a], 1);
            mbar_init(&acc_empty_bar[a], 2 * EPI_WARPS);
        }
        *abort_flag = 0;
        *never_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(static_cast<uint32_t>(TMEM_COLS))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();   // barriers of both CTAs are initialised, tensor memory is allocated
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    bool timed_out = false;

    if (warp == 0) {
        // ------------------------- TMA producer (both CTAs) -------------------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tensorMapA)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tensorMapB)) : "memory");
            int stage = 0;
            uint32_t phase = 0;
            int armed = 0;   // stages loaded and not known to be consumed (for the unwind path)
            for (int t = pair; t < total_tiles && !timed_out; t += pairs) {
                int tm, tn;
                tile_coords(t, tiles_m, tiles_n, tm, tn, GROUP);
                const int n_row = tn * P_::BLOCK + static_cast<int>(rank) * P_::HALF;
                const int m_row = tm * P_::BLOCK + static_cast<int>(rank) * P_::HALF;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait_bounded_sleepy(&empty_bar[stage], phase ^ 1u, abort_flag, 40)) {
                        timed_out = true;
                        break;
                    }
                    unsigned char* p_dst = ring + stage * P_::STAGE_BYTES;
                    unsigned char* q_dst = p_dst + P_::HALF_BYTES;
                    const uint32_t leader_full = cluster_addr(&full_bar[stage], 0);
                    if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * P_::STAGE_BYTES);  // both CTAs' bytes
                    tma_load_2d_pair(p_dst, &tensorMapB, kb * BLOCK_K, n_row, leader_full);
                    tma_load_2d_pair(q_dst, &tensorMapA, kb * BLOCK_K, m_row, leader_full);
                    armed = armed < STAGES ? armed + 1 : STAGES;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (timed_out || *abort_flag) drain_pair_loads(full_bar, stage, phase, armed, STAGES, leader, never_flag);
        }
    } else if (warp == 1) {
        // ------------------------- MMA issuer (leader only) -------------------------
        if (leader && lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            for (int t = pair; t < total_tiles && !timed_out; t += pairs) {
                if (!mbar_wait_bounded(&acc_empty_bar[acc], acc_phase ^ 1u, abort_flag)) {
                    timed_out = true;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * P_::BLOCK);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) {
                        timed_out = true;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t p_addr = smem_u32(ring + stage * P_::STAGE_BYTES);
                    const uint64_t p_desc = smem_desc_k_sw128(p_addr);
                    const uint64_t q_desc = smem_desc_k_sw128(p_addr + P_::HALF_BYTES);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
                        umma_bf16_pair(d_tmem, p_desc + 2u * k, q_desc + 2u * k, IDESC, (kb | k) != 0 ? 1u : 0u);
                    umma_commit_pair(cluster_addr(&empty_bar[stage], 0));   // frees the stage in this CTA ...
                    umma_commit_pair(cluster_addr(&empty_bar[stage], 1));   // ... and in the other one
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (timed_out) break;
                umma_commit_pair(cluster_addr(&acc_full_bar[acc], 0));
                umma_commit_pair(cluster_addr(&acc_full_bar[acc], 1));
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ------------------------- epilogue warps (both CTAs) -------------------------
        const int quarter = warp & 3;
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int t = pair; t < total_tiles; t += pairs) {
            int tm, tn;
            tile_coords(t, tiles_m, tiles_n, tm, tn, GROUP);
            // One lane polls, with sleeps in between (the wait lasts most of a tile's main loop);
            // the other 31 lanes block at the vote.
            const bool ready = lane != 0 || mbar_wait_bounded_sleepy(&acc_full_bar[acc], acc_phase, abort_flag, 200);
            if (!__all_sync(0xffffffffu, ready)) {
                timed_out = true;
                break;
            }
            tc_fence_after();
            // 32 rows x 64 columns at a time through shared memory (16-byte chunks XOR-swizzled by
            // row), so that every store instruction writes four whole 128-byte lines.
            const size_t n_warp = static_cast<size_t>(tn) * P_::BLOCK + rank * P_::HALF + quarter * 32;
            __nv_bfloat16* c_warp = C + n_warp * static_cast<size_t>(M) + static_cast<size_t>(tm) * P_::BLOCK;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(acc * P_::BLOCK);
            unsigned char* stage_buf = epi_smem + (warp - 2) * P_::EPI_WARP_BYTES;
            for (int c0 = 0; c0 < P_::BLOCK; c0 += 64) {
                uint32_t r0[32], r1[32];
                tmem_ld_32cols(t_row + c0, r0);
                tmem_ld_32cols(t_row + c0 + 32, r1);
                tmem_ld_wait();
#pragma unroll
                for (int ch = 0; ch < 8; ++ch) {
                    const uint32_t* r = ch < 4 ? &r0[8 * ch] : &r1[8 * (ch - 4)];
                    uint4 o;
                    o.x = pack_bf16(r[0], r[1]);
                    o.y = pack_bf16(r[2], r[3]);
                    o.z = pack_bf16(r[4], r[5]);
                    o.w = pack_bf16(r[6], r[7]);
                    *reinterpret_cast<uint4*>(stage_buf + lane * 128 + ((ch ^ (lane & 7)) << 4)) = o;
                }
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int row = 4 * j + (lane >> 3);
                    const int ch = lane & 7;
                    const uint4 v = *reinterpret_cast<const uint4*>(stage_buf + row * 128 + ((ch ^ (row & 7)) << 4));
                    *reinterpret_cast<uint4*>(c_warp + static_cast<size_t>(row) * M + c0 + ch * 8) = v;
                }
                __syncwarp();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(cluster_addr(&acc_empty_bar[acc], 0));  // the leader's barrier
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
    }

    if (timed_out) {
        *abort_flag = 1;
        raise_device_status(DEV_GEMM_PIPE_TIMEOUT);
    }
    __syncwarp();
    tc_fence_before();
    cluster_sync_all();   // nobody leaves while the other CTA may still read its operands or signal its barriers
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(static_cast<uint32_t>(TMEM_COLS))
                     : "memory");
    }
}

// ============================================================================
// Two-CTA, two-row-block form: each CTA of the pair owns TWO 128-row n blocks, so the
// pair computes 512 (n) x 256 (m) per tile and each m-side operand byte staged in
// shared memory feeds two MMAs instead of one (48 KB per stage for 2 x 128 x 256 x 64
// MACs per CTA, against 32 KB for half of that in the form above).  Shared-memory and
// L2 traffic per flop drop by a quarter, which is what lets the tensor pipe stay busy.
// The two accumulators take all 512 tensor-memory columns, so they cannot be
// double-buffered.  Instead the part of the epilogue that holds tensor memory is kept
// short: eight epilogue warps, two per lane quarter, one accumulator each, first move
// their rows into registers as packed bf16 (128 registers per lane) and hand tensor
// memory back; the next tile's MMAs then run while the rows go through shared memory to
// global memory.  The producer prefetches the next tile's stages throughout.
// Barriers and pairing are as in the kernel above.
// ============================================================================
namespace g16 {
struct WideCfg {
    static constexpr int TILE_N = 512;     // n rows per pair tile (2 CTAs x 2 blocks x 128)
    static constexpr int TILE_M = 256;     // m rows per pair tile
    static constexpr int HALF = 128;
    static constexpr int STAGES = 4;
    static constexpr int EPI_WARPS = 8;
    static constexpr int THREADS = 64 + 32 * EPI_WARPS;
    static constexpr uint32_t BLOCK_BYTES = HALF * BLOCK_K * 2;   // one 128-row operand block
    static constexpr uint32_t STAGE_BYTES = 3 * BLOCK_BYTES;      // P0, P1, Q half
    static constexpr uint32_t BAR_BYTES = 256;                    // barriers, TMEM slot, abort flag
    // The ring re-cut for the pieces of a filled last wave: one n block and the m rows, 32 KB per stage.
    static constexpr int PIECE_STAGES = 6;
    static constexpr uint32_t PIECE_STAGE_BYTES = 2 * BLOCK_BYTES;
    static_assert(PIECE_STAGES * PIECE_STAGE_BYTES == STAGES * STAGE_BYTES, "the two cuts cover the same ring");
    static constexpr uint32_t EPI_WARP_BYTES = 32 * 128;          // 32 rows x 64 bf16 per epilogue warp
    static constexpr size_t SMEM_BYTES =
        1024 + static_cast<size_t>(STAGES) * STAGE_BYTES + BAR_BYTES + EPI_WARPS * EPI_WARP_BYTES;
};
}  // namespace g16

// The work of one CTA pair of the 512 x 256 form: `full` whole tiles (tile = i * pairs + pair), then, with FILL, its share
// of the last, partly filled wave.  Without FILL a pair simply takes every pairs-th tile, and in the last wave the
// pairs beyond the R = tiles mod pairs remaining tiles idle for a whole tile's time.  With FILL every tile of that wave
// is cut into its two 256-row n blocks, which a pair computes on its own (one 256 x 256 MMA per k-step instead of two,
// over all of K, nothing to hand over); the 2 R pieces are dealt round-robin to all pairs, so where 2 R <= pairs the
// wave costs half a tile's time.  A piece accumulates its k-blocks in the order the whole tile does, in the columns of
// tensor memory the whole tile would use for that block, so the results are bit-identical to the unfilled kernel's.
struct PairPlan {
    int full;        // whole tiles
    int pieces;      // pieces of the last wave that this pair computes
    int wave_first;  // first tile of the last wave
};

template <bool FILL>
__host__ __device__ __forceinline__ PairPlan make_pair_plan(int pair, int pairs, int total_tiles) {
    PairPlan p;
    p.pieces = 0;
    p.wave_first = total_tiles;
    if (!FILL) {
        p.full = pair < total_tiles ? (total_tiles - pair + pairs - 1) / pairs : 0;
    } else {
        p.full = total_tiles / pairs;
        p.wave_first = p.full * pairs;
        const int all = (total_tiles - p.wave_first) * 2;
        p.pieces = pair < all ? (all - pair + pairs - 1) / pairs : 0;
    }
    return p;
}

// Item i of a pair: a tile and which n block of it (-1 = the whole tile).
__host__ __device__ __forceinline__ void plan_item(const PairPlan& p, int i, int pair, int pairs, int& tile, int& blk) {
    if (i < p.full) {
        tile = i * pairs + pair;
        blk = -1;
    } else {
        const int q = pair + (i - p.full) * pairs;
        tile = p.wave_first + q / 2;
        blk = q % 2;
    }
}

// 512 x 256 tiles: each CTA of the pair holds two 128-row n blocks (two accumulators of 256 columns, all of tensor
// memory) against the pair's 256 m rows, so the m-side operand is read once for two MMAs.  Persistent: pair p takes
// tiles p, p + pairs, ... (and, with FILL, pieces of the last wave: see PairPlan).  For the pieces the ring is
// re-cut from four 48 KB stages into six of 32 KB with barriers of their own, so that a piece, which needs 1.33 x the
// operand bytes per MMA cycle, has as many MMA cycles of loads in flight as the 256 x 256 pair kernel has; the
// producer switches over once every stage of the first cut has been consumed.
template <int GROUP, bool FILL>
__device__ __forceinline__ void pair_wide_body(int M, int N, int K, __nv_bfloat16* C, const CUtensorMap* tensorMapA,
                                               const CUtensorMap* tensorMapB) {
    using namespace g16;
    using W_ = WideCfg;
    constexpr int STAGES = W_::STAGES;
    constexpr int PSTAGES = W_::PIECE_STAGES;
    constexpr uint32_t IDESC = instr_desc(256, W_::TILE_M);       // 256 n rows across the pair per MMA, 256 m columns

    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    unsigned char* ring = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(ring + STAGES * W_::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* pfull_bar = empty_bar + STAGES;      // [PSTAGES], the piece ring's (used with FILL only)
    uint64_t* pempty_bar = pfull_bar + PSTAGES;    // [PSTAGES]
    uint64_t* acc_full_bar = pempty_bar + PSTAGES; // [1]
    uint64_t* acc_empty_bar = acc_full_bar + 1;    // [1], only the leader's is used
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* never_flag = tmem_slot + 2;  // stays 0: lets the unwind path wait although abort is set
    unsigned char* epi_smem = ring + STAGES * W_::STAGE_BYTES + W_::BAR_BYTES;   // 128-byte aligned

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1;
    const int pairs = gridDim.x >> 1;
    const int tiles_m = M / W_::TILE_M;
    const int tiles_n = N / W_::TILE_N;
    const int total_tiles = tiles_m * tiles_n;
    const int k_blocks = K / BLOCK_K;
    const PairPlan plan = make_pair_plan<FILL>(pair, pairs, total_tiles);
    const int items = plan.full + plan.pieces;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < PSTAGES; ++s) {
            mbar_init(&pfull_bar[s], 1);
            mbar_init(&pempty_bar[s], 1);
        }
        mbar_init(acc_full_bar, 1);
        mbar_init(acc_empty_bar, 2 * W_::EPI_WARPS);
        *abort_flag = 0;
        *never_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(static_cast<uint32_t>(TMEM_COLS))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    bool timed_out = false;

    if (warp == 0) {
        // ------------------------- TMA producer (both CTAs) -------------------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tensorMapA)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tensorMapB)) : "memory");
            int stage = 0;
            uint32_t phase = 0;
            int armed = 0;   // stages loaded and not known to be consumed (for the unwind path)
            for (int i = 0; i < plan.full && !timed_out; ++i) {
                int tm, tn;
                tile_coords(i * pairs + pair, tiles_m, tiles_n, tm, tn, GROUP);
                // This CTA's two n blocks and its half of the m rows.
                const int n_row0 = tn * W_::TILE_N + static_cast<int>(rank) * 256;
                const int m_row = tm * W_::TILE_M + static_cast<int>(rank) * W_::HALF;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait_bounded_sleepy(&empty_bar[stage], phase ^ 1u, abort_flag, 40)) {
                        timed_out = true;
                        break;
                    }
                    unsigned char* dst = ring + stage * W_::STAGE_BYTES;
                    const uint32_t leader_full = cluster_addr(&full_bar[stage], 0);
                    if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * W_::STAGE_BYTES);   // both CTAs' bytes
                    tma_load_2d_pair(dst, tensorMapB, kb * BLOCK_K, n_row0, leader_full);
                    tma_load_2d_pair(dst + W_::BLOCK_BYTES, tensorMapB, kb * BLOCK_K, n_row0 + W_::HALF, leader_full);
                    tma_load_2d_pair(dst + 2 * W_::BLOCK_BYTES, tensorMapA, kb * BLOCK_K, m_row, leader_full);
                    armed = armed < STAGES ? armed + 1 : STAGES;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            bool in_pieces = false;
            int pstage = 0, parmed = 0;
            uint32_t pphase = 0;
            if (FILL && plan.pieces > 0 && !timed_out) {
                // Before the ring is cut differently every stage of the first cut must have been consumed: the wait
                // that would precede the next load into each of them.
                for (int s = 0; s < STAGES && !timed_out; ++s) {
                    if (!mbar_wait_bounded_sleepy(&empty_bar[stage], phase ^ 1u, abort_flag, 40)) timed_out = true;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!timed_out) {
                    armed = 0;          // nothing of the first cut is in flight any more
                    in_pieces = true;
                }
                for (int i = plan.full; i < items && !timed_out; ++i) {
                    int t, blk, tm, tn;
                    plan_item(plan, i, pair, pairs, t, blk);
                    tile_coords(t, tiles_m, tiles_n, tm, tn, GROUP);
                    const int n_row = tn * W_::TILE_N + static_cast<int>(rank) * 256 + blk * W_::HALF;
                    const int m_row = tm * W_::TILE_M + static_cast<int>(rank) * W_::HALF;
                    for (int kb = 0; kb < k_blocks; ++kb) {
                        if (!mbar_wait_bounded_sleepy(&pempty_bar[pstage], pphase ^ 1u, abort_flag, 40)) {
                            timed_out = true;
                            break;
                        }
                        unsigned char* dst = ring + pstage * W_::PIECE_STAGE_BYTES;
                        const uint32_t leader_full = cluster_addr(&pfull_bar[pstage], 0);
                        if (leader) mbar_arrive_expect_tx(&pfull_bar[pstage], 2 * W_::PIECE_STAGE_BYTES);
                        tma_load_2d_pair(dst, tensorMapB, kb * BLOCK_K, n_row, leader_full);
                        tma_load_2d_pair(dst + W_::BLOCK_BYTES, tensorMapA, kb * BLOCK_K, m_row, leader_full);
                        parmed = parmed < PSTAGES ? parmed + 1 : PSTAGES;
                        if (++pstage == PSTAGES) {
                            pstage = 0;
                            pphase ^= 1u;
                        }
                    }
                }
            }
            if (timed_out || *abort_flag) {
                if (in_pieces) drain_pair_loads(pfull_bar, pstage, pphase, parmed, PSTAGES, leader, never_flag);
                else drain_pair_loads(full_bar, stage, phase, armed, STAGES, leader, never_flag);
            }
        }
    } else if (warp == 1) {
        // ------------------------- MMA issuer (leader only) -------------------------
        if (leader && lane == 0) {
            int stage = 0, pstage = 0;
            uint32_t phase = 0, pphase = 0;
            uint32_t tile_phase = 0;
            for (int i = 0; i < items && !timed_out; ++i) {
                int t, blk;
                plan_item(plan, i, pair, pairs, t, blk);
                if (!mbar_wait_bounded(acc_empty_bar, tile_phase ^ 1u, abort_flag)) {   // both CTAs drained both accumulators
                    timed_out = true;
                    break;
                }
                tc_fence_after();
                if (!FILL || blk < 0) {
                    for (int kb = 0; kb < k_blocks; ++kb) {
                        if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) {
                            timed_out = true;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t base = smem_u32(ring + stage * W_::STAGE_BYTES);
                        const uint64_t p0_desc = smem_desc_k_sw128(base);
                        const uint64_t p1_desc = smem_desc_k_sw128(base + W_::BLOCK_BYTES);
                        const uint64_t q_desc = smem_desc_k_sw128(base + 2 * W_::BLOCK_BYTES);
#pragma unroll
                        for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                            const uint32_t accumulate = (kb | k) != 0 ? 1u : 0u;
                            umma_bf16_pair(tmem_base, p0_desc + 2u * k, q_desc + 2u * k, IDESC, accumulate);
                            umma_bf16_pair(tmem_base + 256u, p1_desc + 2u * k, q_desc + 2u * k, IDESC, accumulate);
                        }
                        umma_commit_pair(cluster_addr(&empty_bar[stage], 0));
                        umma_commit_pair(cluster_addr(&empty_bar[stage], 1));
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                } else {
                    // a piece accumulates in the half of tensor memory that the whole tile would use for its n block
                    const uint32_t d_piece = tmem_base + static_cast<uint32_t>(blk * 256);
                    for (int kb = 0; kb < k_blocks; ++kb) {
                        if (!mbar_wait_bounded(&pfull_bar[pstage], pphase, abort_flag)) {
                            timed_out = true;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t base = smem_u32(ring + pstage * W_::PIECE_STAGE_BYTES);
                        const uint64_t p_desc = smem_desc_k_sw128(base);
                        const uint64_t q_desc = smem_desc_k_sw128(base + W_::BLOCK_BYTES);
#pragma unroll
                        for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
                            umma_bf16_pair(d_piece, p_desc + 2u * k, q_desc + 2u * k, IDESC, (kb | k) != 0 ? 1u : 0u);
                        umma_commit_pair(cluster_addr(&pempty_bar[pstage], 0));
                        umma_commit_pair(cluster_addr(&pempty_bar[pstage], 1));
                        if (++pstage == PSTAGES) {
                            pstage = 0;
                            pphase ^= 1u;
                        }
                    }
                }
                if (timed_out) break;
                umma_commit_pair(cluster_addr(acc_full_bar, 0));
                umma_commit_pair(cluster_addr(acc_full_bar, 1));
                tile_phase ^= 1u;
            }
        }
    } else {
        // ------------------------- epilogue warps (both CTAs) -------------------------
        // Warps 2-9: warp index mod 4 picks the 32-lane quarter of tensor memory it can reach;
        // the two warps of a quarter take one accumulator (n block) each.
        const int quarter = warp & 3;
        const int block = (warp - 2) >> 2;
        uint32_t tile_phase = 0;
        for (int i = 0; i < items; ++i) {
            int t, blk, tm, tn;
            plan_item(plan, i, pair, pairs, t, blk);
            tile_coords(t, tiles_m, tiles_n, tm, tn, GROUP);
            const bool ready = lane != 0 || mbar_wait_bounded_sleepy(acc_full_bar, tile_phase, abort_flag, 200);
            if (!__all_sync(0xffffffffu, ready)) {
                timed_out = true;
                break;
            }
            tc_fence_after();
            if (FILL && blk >= 0 && blk != block) {
                // The other n block's warps drain this piece.  This warp has waited for it like everybody (which keeps
                // it in step with the barrier's phases) and hands its share of tensor memory back at once.
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(cluster_addr(acc_empty_bar, 0));
                tile_phase ^= 1u;
                continue;
            }
            // A lane reads one accumulator row (one n, consecutive m).  Writing that row straight to
            // global memory would make every store instruction touch 32 different lines, 16 bytes
            // each; instead the warp passes 32 rows x 64 columns at a time through shared memory
            // (16-byte chunks XOR-swizzled by row, conflict-free both ways) and stores whole
            // 128-byte lines: 4 rows per instruction.
            const size_t n_warp = static_cast<size_t>(tn) * W_::TILE_N + rank * 256 + block * W_::HALF + quarter * 32;
            __nv_bfloat16* c_warp = C + n_warp * static_cast<size_t>(M) + static_cast<size_t>(tm) * W_::TILE_M;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(block * 256);
            unsigned char* stage_buf = epi_smem + (warp - 2) * W_::EPI_WARP_BYTES;
            // The whole accumulator row first goes into registers as packed bf16 (256 columns = 128
            // registers), so that tensor memory can be handed back and the next tile's MMAs start
            // while this tile is still on its way to global memory.
            uint32_t packed[W_::TILE_M / 2];
#pragma unroll
            for (int c0 = 0; c0 < W_::TILE_M; c0 += 32) {
                uint32_t r[32];
                tmem_ld_32cols(t_row + c0, r);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 16; ++e) packed[c0 / 2 + e] = pack_bf16(r[2 * e], r[2 * e + 1]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(cluster_addr(acc_empty_bar, 0));
#pragma unroll
            for (int c0 = 0; c0 < W_::TILE_M; c0 += 64) {
#pragma unroll
                for (int ch = 0; ch < 8; ++ch) {
                    uint4 o;
                    o.x = packed[c0 / 2 + 4 * ch + 0];
                    o.y = packed[c0 / 2 + 4 * ch + 1];
                    o.z = packed[c0 / 2 + 4 * ch + 2];
                    o.w = packed[c0 / 2 + 4 * ch + 3];
                    *reinterpret_cast<uint4*>(stage_buf + lane * 128 + ((ch ^ (lane & 7)) << 4)) = o;
                }
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int row = 4 * j + (lane >> 3);
                    const int ch = lane & 7;
                    const uint4 v = *reinterpret_cast<const uint4*>(stage_buf + row * 128 + ((ch ^ (row & 7)) << 4));
                    *reinterpret_cast<uint4*>(c_warp + static_cast<size_t>(row) * M + c0 + ch * 8) = v;
                }
                __syncwarp();
            }
            tile_phase ^= 1u;
        }
    }

    if (timed_out) {
        *abort_flag = 1;
        raise_device_status(DEV_GEMM_PIPE_TIMEOUT);
    }
    __syncwarp();
    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(static_cast<uint32_t>(TMEM_COLS))
                     : "memory");
    }
}

template <int GROUP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(g16::WideCfg::THREADS, 1)
cutlass_my_h100_match_no_tail_pair_wide(int M, int N, int K, __nv_bfloat16* C,
                                        const __grid_constant__ CUtensorMap tensorMapA,
                                        const __grid_constant__ CUtensorMap tensorMapB) {
    pair_wide_body<GROUP, false>(M, N, K, C, &tensorMapA, &tensorMapB);
}

// The same kernel with the tiles of the last, partly filled wave cut into their two n blocks, dealt to all CTA pairs.
template <int GROUP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(g16::WideCfg::THREADS, 1)
cutlass_my_h100_match_no_tail_pair_wide_fill(int M, int N, int K, __nv_bfloat16* C,
                                             const __grid_constant__ CUtensorMap tensorMapA,
                                             const __grid_constant__ CUtensorMap tensorMapB) {
    pair_wide_body<GROUP, true>(M, N, K, C, &tensorMapA, &tensorMapB);
}

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

std::mutex g_map_mu;
EncodeTiledFn g_encode = nullptr;

struct MapKey {
    int dev;
    const void* ptr;
    int rows, k, box_rows;
    bool operator==(const MapKey& o) const {
        return dev == o.dev && ptr == o.ptr && rows == o.rows && k == o.k && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = reinterpret_cast<size_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
        h ^= (static_cast<size_t>(k.rows) << 32) ^ static_cast<size_t>(k.k) ^ (static_cast<size_t>(k.box_rows) << 20) ^
             (static_cast<size_t>(k.dev) << 56);
        return h;
    }
};
// A tensor map is a pure function of its key, so a cached entry can never be stale.
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

int get_tensor_map(int dev, const void* ptr, int rows, int k, int box_rows, CUtensorMap* out) {
    std::lock_guard<std::mutex> lk(g_map_mu);
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || !fn || q != cudaDriverEntryPointSuccess)
            return set_error(PRISM_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    const MapKey key{dev, ptr, rows, k, box_rows};
    auto it = g_maps.find(key);
    if (it != g_maps.end()) {
        *out = it->second;
        return PRISM_B200_OK;
    }
    CUtensorMap m;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(g16::BLOCK_K), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(PRISM_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps.emplace(key, m);
    *out = m;
    return PRISM_B200_OK;
}

template <int BLOCK_Q>
int launch_gemm(int dev, int sms, int M, int N, int K, const void* A, const void* B, void* C, cudaStream_t s) {
    using C_ = g16::Cfg<BLOCK_Q>;
    CUtensorMap map_a, map_b;
    if (int rc = get_tensor_map(dev, A, M, K, BLOCK_Q, &map_a)) return rc;
    if (int rc = get_tensor_map(dev, B, N, K, g16::BLOCK_P, &map_b)) return rc;
    auto kern = cutlass_my_h100_match_no_tail<BLOCK_Q>;
    {
        static bool attr_set[64] = {};
        static std::mutex mu;
        std::lock_guard<std::mutex> lk(mu);
        if (dev < 0 || dev >= 64 || !attr_set[dev]) {
            PRISM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                static_cast<int>(C_::SMEM_BYTES)));
            if (dev >= 0 && dev < 64) attr_set[dev] = true;
        }
    }
    const int tiles = (M / BLOCK_Q) * (N / g16::BLOCK_P);
    const int grid = tiles < sms ? tiles : sms;
    kern<<<grid, g16::THREADS, C_::SMEM_BYTES, s>>>(M, N, K, static_cast<__nv_bfloat16*>(C), map_a, map_b);
    PRISM_CUDA_TRY(cudaGetLastError());
    count_launch();
    return PRISM_B200_OK;
}

// The one-CTA kernel with the scaling epilogue: D = alpha * A * B^T + beta * Cin.
template <int BLOCK_Q>
int launch_gemm_axpby(int dev, int sms, int M, int N, int K, float alpha, const void* A, const void* B, float beta,
                      const void* Cin, void* D, cudaStream_t s) {
    using C_ = g16::Cfg<BLOCK_Q>;
    CUtensorMap map_a, map_b;
    if (int rc = get_tensor_map(dev, A, M, K, BLOCK_Q, &map_a)) return rc;
    if (int rc = get_tensor_map(dev, B, N, K, g16::BLOCK_P, &map_b)) return rc;
    auto kern = cutlass_my_h100_match_no_tail_axpby<BLOCK_Q>;
    {
        static bool attr_set[64] = {};
        static std::mutex mu;
        std::lock_guard<std::mutex> lk(mu);
        if (dev < 0 || dev >= 64 || !attr_set[dev]) {
            PRISM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                static_cast<int>(C_::SMEM_BYTES)));
            if (dev >= 0 && dev < 64) attr_set[dev] = true;
        }
    }
    const int tiles = (M / BLOCK_Q) * (N / g16::BLOCK_P);
    const int grid = tiles < sms ? tiles : sms;
    kern<<<grid, g16::THREADS, C_::SMEM_BYTES, s>>>(M, N, K, static_cast<__nv_bfloat16*>(D), map_a, map_b, alpha, beta,
                                                    static_cast<const __nv_bfloat16*>(Cin));
    PRISM_CUDA_TRY(cudaGetLastError());
    count_launch();
    return PRISM_B200_OK;
}

using PairKernel = void (*)(int, int, int, __nv_bfloat16*, const CUtensorMap, const CUtensorMap);

std::mutex g_launch_mu;   // guards the per-device caches below; entry points may be called from several host threads

void pair_launch_config(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int threads, size_t smem, cudaStream_t s) {
    *cfg = cudaLaunchConfig_t{};
    cfg->blockDim = dim3(static_cast<unsigned>(threads));
    cfg->dynamicSmemBytes = smem;
    cfg->stream = s;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg->attrs = attr;
    cfg->numAttrs = 1;
}

// CTA pairs of `kern` that the device holds at once, found once per device and kernel (`cache` is the
// kernel's own table); also raises the kernel's dynamic shared-memory limit.
template <typename Kernel>
int pair_capacity(Kernel kern, int* cache, int threads, size_t smem, int dev, int* out) {
    std::lock_guard<std::mutex> lk(g_launch_mu);
    const bool cacheable = dev >= 0 && dev < 64;
    if (cacheable && cache[dev]) {
        *out = cache[dev];
        return PRISM_B200_OK;
    }
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    pair_launch_config(&cfg, attr, threads, smem, nullptr);
    PRISM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    int sms = 0;
    PRISM_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    cfg.gridDim = dim3(static_cast<unsigned>(sms / 2 * 2));
    int clusters = 0;
    PRISM_CUDA_TRY(cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg));
    if (clusters < 1) return set_error(PRISM_B200_ERR_CUDA, "gemm_bf16: no 2-CTA cluster fits on this device");
    if (cacheable) cache[dev] = clusters;
    *out = clusters;
    return PRISM_B200_OK;
}

// Launches one of the two-CTA kernels: persistent, as many pairs as the device holds at once.
int launch_pair_kernel(PairKernel kern, int* cache, int threads, size_t smem, int tiles, int dev, int M, int N,
                       int K, const CUtensorMap& map_a, const CUtensorMap& map_b, void* C, cudaStream_t s) {
    int pairs_cap = 0;
    if (int rc = pair_capacity(kern, cache, threads, smem, dev, &pairs_cap)) return rc;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    pair_launch_config(&cfg, attr, threads, smem, s);
    const int pairs = tiles < pairs_cap ? tiles : pairs_cap;
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
    PRISM_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, M, N, K, static_cast<__nv_bfloat16*>(C), map_a, map_b));
    count_launch();
    return PRISM_B200_OK;
}

// m-tiles walked per n-tile: 8 for the 256 x 256 pair tiles, 16 for the 512 x 256 ones
// (measured best of 4 / 8 / 16 / 32 at 8192^3 on a B200).
int launch_gemm_pair(int dev, int M, int N, int K, const void* A, const void* B, void* C, cudaStream_t s) {
    using P_ = g16::PairCfg;
    CUtensorMap map_a, map_b;
    if (int rc = get_tensor_map(dev, A, M, K, P_::HALF, &map_a)) return rc;
    if (int rc = get_tensor_map(dev, B, N, K, P_::HALF, &map_b)) return rc;
    static int max_pairs[64] = {};
    return launch_pair_kernel(cutlass_my_h100_match_no_tail_pair<8>, max_pairs, g16::THREADS, P_::SMEM_BYTES,
                              (M / P_::BLOCK) * (N / P_::BLOCK), dev, M, N, K, map_a, map_b, C, s);
}

// ---- the 512 x 256 form and the filling of its last wave ---------------------------------------
bool g_fill_mode_set = false;   // prism_b200_gemm_bf16_fill_mode was called: the environment no longer decides
int g_fill_mode = -1;           // -1 by shape, 0 never, 2 whenever the last wave is partly filled

// Main-loop throughput of a piece (one 256 x 256 MMA per k-step on 32 KB of operands per CTA) relative to a whole
// 512 x 256 tile's, measured on a B200.
constexpr double kPieceEff = 0.92;

// Time of the 512 x 256 form in units of one whole tile, and whether the tiles of the last wave are cut into their two
// n blocks to reach it (*fill).  By shape, a fill is taken where it halves the last wave (2 R <= pairs).
double wide_form_time(long long tiles, int pairs, int mode, bool* fill) {
    const long long waves = tiles / pairs;
    const int rem = static_cast<int>(tiles % pairs);
    bool cut = false;
    double last = rem ? 1.0 : 0.0;
    if (rem && mode != 0) {
        const double pieces = static_cast<double>((2 * rem + pairs - 1) / pairs) / 2.0 / kPieceEff;
        if (mode == 2 || pieces < 0.9) {
            cut = true;
            last = pieces;
        }
    }
    if (fill) *fill = cut;
    return static_cast<double>(waves) + last;
}

int launch_gemm_pair_wide(int dev, int M, int N, int K, const void* A, const void* B, void* C, cudaStream_t s) {
    using W_ = g16::WideCfg;
    CUtensorMap map_a, map_b;
    if (int rc = get_tensor_map(dev, A, M, K, W_::HALF, &map_a)) return rc;
    if (int rc = get_tensor_map(dev, B, N, K, W_::HALF, &map_b)) return rc;
    static int max_pairs[64] = {}, max_pairs_fill[64] = {};
    const int tiles = (M / W_::TILE_M) * (N / W_::TILE_N);
    int pairs_cap = 0;
    if (int rc = pair_capacity(cutlass_my_h100_match_no_tail_pair_wide_fill<16>, max_pairs_fill, W_::THREADS, W_::SMEM_BYTES,
                               dev, &pairs_cap))
        return rc;
    bool fill = false;
    (void)wide_form_time(tiles, pairs_cap, g_fill_mode, &fill);
    if (fill) {
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[1];
        pair_launch_config(&cfg, attr, W_::THREADS, W_::SMEM_BYTES, s);
        // every pair that has a tile or a piece: all of them once there is a full wave
        const long long items = static_cast<long long>(tiles / pairs_cap) * pairs_cap + 2LL * (tiles % pairs_cap);
        const int pairs = items < pairs_cap ? static_cast<int>(items) : pairs_cap;
        cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
        PRISM_CUDA_TRY(cudaLaunchKernelEx(&cfg, cutlass_my_h100_match_no_tail_pair_wide_fill<16>, M, N, K,
                                          static_cast<__nv_bfloat16*>(C), map_a, map_b));
        count_launch();
        return PRISM_B200_OK;
    }
    return launch_pair_kernel(cutlass_my_h100_match_no_tail_pair_wide<16>, max_pairs, W_::THREADS, W_::SMEM_BYTES, tiles, dev,
                              M, N, K, map_a, map_b, C, s);
}

}  // namespace
}  // namespace prism_b200

using namespace prism_b200;

extern "C" int prism_b200_gemm_bf16_fill_mode(int mode) {
    if (mode != -1 && mode != 0 && mode != 2)
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "gemm_bf16_fill_mode: -1, 0 or 2");
    std::lock_guard<std::mutex> lk(g_launch_mu);
    g_fill_mode_set = true;
    g_fill_mode = mode;
    return PRISM_B200_OK;
}

extern "C" int prism_b200_gemm_bf16_fill_plan(int tiles, int pairs, int fill, int pair, int capacity, int* tile_block,
                                              int* count) {
    if (!count || tiles < 0 || pairs < 1 || (fill != 0 && fill != 1) || pair < 0 || pair >= pairs || capacity < 0 ||
        (capacity > 0 && !tile_block))
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "gemm_bf16_fill_plan: bad argument");
    const PairPlan p = fill ? make_pair_plan<true>(pair, pairs, tiles) : make_pair_plan<false>(pair, pairs, tiles);
    const int items = p.full + p.pieces;
    for (int i = 0; i < items && i < capacity; ++i) plan_item(p, i, pair, pairs, tile_block[2 * i], tile_block[2 * i + 1]);
    *count = items;
    return PRISM_B200_OK;
}

extern "C" int prism_b200_gemm_bf16_axpby(int M, int N, int K, float alpha, const uint16_t* A, const uint16_t* B, float beta,
                                          const uint16_t* Cin, uint16_t* D, void* stream) {
    if (M < 0 || N < 0 || K < 0) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "gemm_bf16_axpby: negative dimension");
    if (M == 0 || N == 0) return PRISM_B200_OK;
    if (!A || !B || !Cin || !D) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "gemm_bf16_axpby: null pointer");
    if (M % 128 || N % 128 || K % 64 || K == 0)
        return set_error(PRISM_B200_ERR_UNSUPPORTED_SHAPE,
                         "gemm_bf16_axpby: need M %% 128 == 0, N %% 128 == 0, K %% 64 == 0, K > 0 (got %d, %d, %d)", M, N, K);
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(Cin) |
         reinterpret_cast<uintptr_t>(D)) & 15u)
        return set_error(PRISM_B200_ERR_MISALIGNED, "gemm_bf16_axpby: A, B, Cin and D must be 16-byte aligned");
    if (Cin != D) {
        const uintptr_t a = reinterpret_cast<uintptr_t>(Cin), b = reinterpret_cast<uintptr_t>(D);
        const size_t bytes = static_cast<size_t>(M) * N * 2;
        if (a < b + bytes && b < a + bytes)
            return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "gemm_bf16_axpby: Cin and D overlap without being equal");
    }
    if (int rc = bind_status_word()) return rc;
    int dev = 0, sms = 0;
    PRISM_CUDA_TRY(cudaGetDevice(&dev));
    PRISM_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // 256-wide m-tiles unless M does not divide or they would leave a poorly filled last wave (as in prism_b200_gemm_bf16).
    bool wide = (M % 256 == 0);
    if (wide) {
        auto eff = [&](int tiles) { return static_cast<double>(tiles) / (((tiles + sms - 1) / sms) * sms); };
        if (eff((M / 256) * (N / 128)) + 0.10 < eff((M / 128) * (N / 128))) wide = false;
    }
    return wide ? launch_gemm_axpby<256>(dev, sms, M, N, K, alpha, A, B, beta, Cin, D, s)
                : launch_gemm_axpby<128>(dev, sms, M, N, K, alpha, A, B, beta, Cin, D, s);
}

extern "C" int prism_b200_gemm_bf16(int M, int N, int K, const uint16_t* A, const uint16_t* B, uint16_t* C,
                                    void* stream) {
    if (M < 0 || N < 0 || K < 0) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "gemm_bf16: negative dimension");
    if (M == 0 || N == 0) return PRISM_B200_OK;
    if (!A || !B || !C) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "gemm_bf16: null pointer");
    if (M % 128 || N % 128 || K % 64 || K == 0)
        return set_error(PRISM_B200_ERR_UNSUPPORTED_SHAPE,
                         "gemm_bf16: need M %% 128 == 0, N %% 128 == 0, K %% 64 == 0, K > 0 (got %d, %d, %d)", M, N, K);
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15u)
        return set_error(PRISM_B200_ERR_MISALIGNED, "gemm_bf16: A, B and C must be 16-byte aligned");
    if (int rc = bind_status_word()) return rc;
    int dev = 0;
    PRISM_CUDA_TRY(cudaGetDevice(&dev));
    int sms = 0;
    static int forced = -1;
    {
        static int sm_count[64] = {};
        static bool env_read = false;
        std::lock_guard<std::mutex> lk(g_launch_mu);
        sms = (dev >= 0 && dev < 64) ? sm_count[dev] : 0;
        if (sms == 0) {
            PRISM_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
            if (dev >= 0 && dev < 64) sm_count[dev] = sms;
        }
        if (!env_read) {
            // PRISM_B200_GEMM_PAIR = 0 / 1 / 2 forces one-CTA / 256 x 256 pair / 512 x 256 pair,
            // PRISM_B200_GEMM_FILL = 0 / 2 the 512 x 256 form without / with its partly filled last wave cut in pieces (tests)
            const char* e = getenv("PRISM_B200_GEMM_PAIR");
            forced = e ? atoi(e) : -1;
            const char* fm = getenv("PRISM_B200_GEMM_FILL");
            if (!g_fill_mode_set && fm) {
                const int v = atoi(fm);
                g_fill_mode = (v == 0 || v == 2) ? v : -1;
            }
            env_read = true;
        }
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    {
        // Which form: estimated main-loop time in units of one 128 x 256 tile on one SM, waves x
        // tile size / (measured relative efficiency of the form).  Small problems (under 2^35
        // multiply-adds) stay with the one-CTA forms, whose launch costs less.
        const bool pair_ok = M % 256 == 0 && N % 256 == 0;
        const bool wide_ok = M % 256 == 0 && N % 512 == 0;
        int form = 0;  // 0 one CTA, 1 pair, 2 wide pair
        if (forced >= 0) {
            form = (forced == 2 && wide_ok) ? 2 : (forced == 1 && pair_ok) ? 1 : 0;
        } else if (static_cast<double>(M) * N * K >= 34359738368.0) {
            const int pairs = sms / 2 > 0 ? sms / 2 : 1;
            auto waves = [](long long tiles, int slots) { return static_cast<double>((tiles + slots - 1) / slots); };
            const double t_single = waves(static_cast<long long>(M / 128) * (N / 128), sms) * 0.5 / 0.75;
            double best = t_single;
            if (M % 256 == 0) {
                const double t = waves(static_cast<long long>(M / 256) * (N / 128), sms) / 0.93;
                if (t < best) best = t;
            }
            if (pair_ok) {
                const double t = waves(static_cast<long long>(M / 256) * (N / 256), pairs) / 0.97;
                if (t < best) { best = t; form = 1; }
            }
            if (wide_ok) {
                const double t = wide_form_time(static_cast<long long>(M / 256) * (N / 512), pairs, g_fill_mode, nullptr) * 2.0;
                if (t <= best) { best = t; form = 2; }
            }
        }
        if (form == 2) return launch_gemm_pair_wide(dev, M, N, K, A, B, C, s);
        if (form == 1) return launch_gemm_pair(dev, M, N, K, A, B, C, s);
    }
    // 256-wide m-tiles halve the operand traffic per flop; fall back to 128 when M
    // does not divide or when the wider tile would leave a poorly filled last wave.
    bool wide = (M % 256 == 0);
    if (wide) {
        auto eff = [&](int tiles) { return static_cast<double>(tiles) / (((tiles + sms - 1) / sms) * sms); };
        const int t256 = (M / 256) * (N / 128), t128 = (M / 128) * (N / 128);
        if (eff(t256) + 0.10 < eff(t128)) wide = false;
    }
    return wide ? launch_gemm<256>(dev, sms, M, N, K, A, B, C, s) : launch_gemm<128>(dev, sms, M, N, K, A, B, C, s);
}
