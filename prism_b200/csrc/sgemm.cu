// FP32 SGEMM family for B200, C = alpha * A * B + beta * C, row-major, pure FFMA
// (no TF32, no tensor cores).
//
// The entry points keep the parameter lists of the emitted reference kernels
// (generated/my_sgemm_kernel_{1,2,3,4,5}.cu, generated/sgemm_shared_mem_block.cu):
//   (int M, int N, int K, float alpha, [const] float* A, [const] float* B,
//    float beta, float* C, int <block_size | tile_size | num_blocks_N>)
// with a 1-D grid and a linear block id, and the host dispatcher mirrors
// `run_my_kernel` (evals/4090_sgemm/runner.cu:245-267).
//
// Kernels 1-4 and 6 are the small rungs of the ladder.  Kernel 5 is the one that
// matters for throughput: the A slice is transposed on its way into shared memory
// (coalesced 16-byte loads, k-major stores), the B slice arrives by cp.async, and
// four warps run an 8x16 register tile per lane on packed fma.rn.f32x2.
#include "common.cuh"

#include <mutex>

namespace prism_b200 {

// ============================================================================
// Kernel 1: one thread per element of C (generated/my_sgemm_kernel_1.cu:1-28).
// The reference has no bounds check and needs M*N to be a multiple of the block
// size; this one guards the tail.
// ============================================================================
__global__ void my_sgemm_kernel_1(int M, int N, int K, float alpha, const float* A, const float* B, float beta,
                                  float* C, int block_size) {
    const long long tid = static_cast<long long>(blockIdx.x) * block_size + threadIdx.x;
    if (tid >= static_cast<long long>(M) * N) return;
    const int row = static_cast<int>(tid / N);
    const int col = static_cast<int>(tid % N);
    const float* a = A + static_cast<size_t>(row) * K;
    const float* b = B + col;
    float acc = 0.f;
    for (int k = 0; k < K; ++k) acc = fmaf(a[k], b[static_cast<size_t>(k) * N], acc);
    float* c = C + static_cast<size_t>(row) * N + col;
    *c = alpha * acc + beta * *c;
}

// ============================================================================
// Kernel 2: same dot product, threads mapped through tile_size x tile_size tiles
// so that a warp walks along a row of C (generated/my_sgemm_kernel_2.cu:1-32).
// ============================================================================
__global__ void my_sgemm_kernel_2(int M, int N, int K, float alpha, const float* A, const float* B, float beta,
                                  float* C, int tile_size) {
    const long long gtid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int per_tile = tile_size * tile_size;
    const int tiles_per_row = (N + tile_size - 1) / tile_size;
    const long long tile = gtid / per_tile;
    const int local = static_cast<int>(gtid % per_tile);
    const long long row = (tile / tiles_per_row) * tile_size + local / tile_size;
    const long long col = (tile % tiles_per_row) * tile_size + local % tile_size;
    if (row >= M || col >= N) return;
    const float* a = A + row * K;
    const float* b = B + col;
    float acc = 0.f;
    for (int k = 0; k < K; ++k) acc = fmaf(a[k], b[static_cast<size_t>(k) * N], acc);
    float* c = C + row * N + col;
    *c = alpha * acc + beta * *c;
}

// ============================================================================
// Kernel 3 of the evaluation: BLOCKSIZE x BLOCKSIZE shared-memory tiles, one
// output per thread (generated/sgemm_shared_mem_block.cu:1-49).  Dimensions
// must be multiples of BLOCKSIZE (the dispatcher checks).
// ============================================================================
template <int BLOCKSIZE>
__global__ void __launch_bounds__(BLOCKSIZE* BLOCKSIZE)
sgemm_shared_mem_block(int M, int N, int K, float alpha, const float* A, const float* B, float beta, float* C,
                       int num_blocks_N) {
    __shared__ float As[BLOCKSIZE][BLOCKSIZE];
    __shared__ float Bs[BLOCKSIZE][BLOCKSIZE];
    const int tile_row = blockIdx.x / num_blocks_N;
    const int tile_col = blockIdx.x % num_blocks_N;
    const int tr = threadIdx.x / BLOCKSIZE;
    const int tc = threadIdx.x % BLOCKSIZE;
    const float* a = A + static_cast<size_t>(tile_row * BLOCKSIZE + tr) * K + tc;
    const float* b = B + static_cast<size_t>(tr) * N + tile_col * BLOCKSIZE + tc;
    float acc = 0.f;
    for (int k0 = 0; k0 < K; k0 += BLOCKSIZE) {
        As[tr][tc] = a[k0];
        Bs[tr][tc] = b[static_cast<size_t>(k0) * N];
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BLOCKSIZE; ++k) acc = fmaf(As[tr][k], Bs[k][tc], acc);
        __syncthreads();
    }
    float* c = C + static_cast<size_t>(tile_row * BLOCKSIZE + tr) * N + tile_col * BLOCKSIZE + tc;
    *c = alpha * acc + beta * *c;
}

// ============================================================================
// Kernel 6 (the reference's generated/my_sgemm_kernel_3.cu:1-83, which its
// harness never launches): BM x BN tile, TM x TN outputs per thread, scalar
// accesses.  Here every access is bounds-checked, so it doubles as the kernel
// for shapes that the faster kernels do not divide.
// ============================================================================
template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM * BN) / (TM * TN))
my_sgemm_kernel_3(int M, int N, int K, float alpha, const float* A, const float* B, float beta, float* C,
                  int num_blocks_N) {
    constexpr int THREADS = (BM * BN) / (TM * TN);
    __shared__ float As[BK][BM + 1];  // k-major so a thread's TM rows are contiguous
    __shared__ float Bs[BK][BN];
    const int row0 = (blockIdx.x / num_blocks_N) * BM;
    const int col0 = (blockIdx.x % num_blocks_N) * BN;
    const int ty = threadIdx.x / (BN / TN);
    const int tx = threadIdx.x % (BN / TN);
    float acc[TM][TN] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int e = threadIdx.x; e < BM * BK; e += THREADS) {
            const int r = e / BK, k = e % BK;
            const int gr = row0 + r, gk = k0 + k;
            As[k][r] = (gr < M && gk < K) ? A[static_cast<size_t>(gr) * K + gk] : 0.f;
        }
        for (int e = threadIdx.x; e < BK * BN; e += THREADS) {
            const int k = e / BN, c = e % BN;
            const int gk = k0 + k, gc = col0 + c;
            Bs[k][c] = (gk < K && gc < N) ? B[static_cast<size_t>(gk) * N + gc] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float ra[TM], rb[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) ra[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) rb[j] = Bs[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ra[i], rb[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gr = row0 + ty * TM + i;
        if (gr >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gc = col0 + tx * TN + j;
            if (gc < N) {
                float* c = C + static_cast<size_t>(gr) * N + gc;
                *c = alpha * acc[i][j] + beta * *c;
            }
        }
    }
}

// ============================================================================
// Kernel 4: 128x128x8 tiles, 8x8 outputs per thread, 128-bit global and shared
// accesses, A transposed on its way into shared memory
// (generated/my_sgemm_kernel_4.cu:1-88).  M, N multiples of BM, BN; K of BK.
// The next k-slice is fetched into registers while the current one is consumed.
// ============================================================================
template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM * BN) / (TM * TN))
my_sgemm_kernel_4(int M, int N, int K, float alpha, float* A, float* B, float beta, float* C, int num_blocks_N) {
    static_assert(BM == 128 && BN == 128 && BK == 8 && TM == 8 && TN == 8, "one 16-byte load per thread per operand");
    __shared__ __align__(16) float As[2][BK][BM];
    __shared__ __align__(16) float Bs[2][BK][BN];
    const int row0 = (blockIdx.x / num_blocks_N) * BM;
    const int col0 = (blockIdx.x % num_blocks_N) * BN;
    const int ty = threadIdx.x / (BN / TN);
    const int tx = threadIdx.x % (BN / TN);
    const int a_row = threadIdx.x / (BK / 4), a_col = (threadIdx.x % (BK / 4)) * 4;
    const int b_row = threadIdx.x / (BN / 4), b_col = (threadIdx.x % (BN / 4)) * 4;
    const float* a_src = A + static_cast<size_t>(row0 + a_row) * K + a_col;
    const float* b_src = B + static_cast<size_t>(b_row) * N + col0 + b_col;

    float acc[TM][TN] = {};
    float4 ra = *reinterpret_cast<const float4*>(a_src);
    float4 rb = *reinterpret_cast<const float4*>(b_src);
    int buf = 0;
    for (int k0 = 0; k0 < K; k0 += BK) {
        As[buf][a_col + 0][a_row] = ra.x;
        As[buf][a_col + 1][a_row] = ra.y;
        As[buf][a_col + 2][a_row] = ra.z;
        As[buf][a_col + 3][a_row] = ra.w;
        *reinterpret_cast<float4*>(&Bs[buf][b_row][b_col]) = rb;
        __syncthreads();
        if (k0 + BK < K) {
            ra = *reinterpret_cast<const float4*>(a_src + k0 + BK);
            rb = *reinterpret_cast<const float4*>(b_src + static_cast<size_t>(k0 + BK) * N);
        }
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float fa[TM], fb[TN];
            // Two 16-byte reads per operand, 64 columns apart, keep each quarter-warp on distinct banks.
            *reinterpret_cast<float4*>(&fa[0]) = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
            *reinterpret_cast<float4*>(&fa[4]) = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
            *reinterpret_cast<float4*>(&fb[0]) = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
            *reinterpret_cast<float4*>(&fb[4]) = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(fa[i], fb[j], acc[i][j]);
        }
        buf ^= 1;  // the other buffer was last read before the barrier above
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = row0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float4* c = reinterpret_cast<float4*>(C + static_cast<size_t>(r) * N + col0 + h * 64 + tx * 4);
            float4 v = *c;
            v.x = alpha * acc[i][h * 4 + 0] + beta * v.x;
            v.y = alpha * acc[i][h * 4 + 1] + beta * v.y;
            v.z = alpha * acc[i][h * 4 + 2] + beta * v.z;
            v.w = alpha * acc[i][h * 4 + 3] + beta * v.w;
            *c = v;
        }
    }
}

// ============================================================================
// Kernel 5: the throughput kernel (generated/my_sgemm_kernel_5.cu:1-84 with
// loadFromGmem_our / processFromSmem_our, evals/4090_sgemm/my_kernel_utils.cuh:13-89).
//
// CTA tile 128 x 128 (or 64 x 128 when there are few tiles), k-slice 16, two shared-memory
// buffers, 128 threads, two CTAs per SM (two warps per scheduler, so a lane may use 255 registers).
//   Staging: the A slice (128 rows x 16 k) is read with coalesced 16-byte loads (four
//     lanes per row) into registers while the current slice is consumed, then stored
//     TRANSPOSED (k-major, row stride 132 floats) into the other buffer, so that a lane's
//     rows for one k are two 16-byte reads and only 8 floats of A are live at a time.  The
//     B slice (16 rows x 512 or 256 B) goes straight to shared memory with 16-byte
//     cp.async, no registers.  One __syncthreads per slice.
//   Compute: 2 x 2 arrangement of 64 x 64 warp tiles.  A lane owns rows
//     wm0 + 4 (lane & 7) + {0..3} and 32 more down, and columns wn0 + 16 j + 4 (lane >> 3) .. +3
//     (j = 0..3): 8 x 16 = 128 accumulators.  Per k it reads 2 x 16 B of A and 4 x 16 B
//     of B (every read a broadcast of distinct contiguous 16-byte chunks) for 128 FMAs.
//     With PACKED the FMAs are issued as fma.rn.f32x2 on column pairs: two independent
//     fp32 FMAs per instruction, the same bits as the scalar form.  All eight duplicated
//     A values are prepared first and the FMAs go column pair by column pair, so that
//     consecutive instructions share their B operand.
//   Measured on a B200 at 4096^3 / 8192^3 (TFLOP/s): this form 63.1 / 64.5; the same with
//     B register-staged 55.9 / 57.3; with B rows brought in by the bulk-copy (TMA) engine onto an
//     mbarrier 57.6 / 59.9; with A through 4-byte cp.async 54.0 / 55.4; k-slices
//     of 8 or 32: 58.9 / 60.4 and 57.9 / 61.5; A loaded one row per lane 56.3 / 57.6; a
//     256-thread form with 8 x 8 outputs per lane 60.5 / 61.8; 256 x 128 tiles with one CTA per
//     SM 52.2 / 60.4.  An earlier form that staged row-major A with cp.async.bulk through a
//     three-stage mbarrier ring reached 51.5 / 53.6: its A fragments (four k per 16-byte
//     read) kept 32 registers live and left the compiler no room to overlap reads and FMAs.
//     A register-only loop of the same fma.rn.f32x2 pattern peaks at 69.3.
// Needs M % 128 == 0, N % 128 == 0, K % 16 == 0 and 16-byte aligned A, B, C.
// ============================================================================
namespace k5 {
constexpr int BM = 128, BN = 128, BK = 16;
constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
}  // namespace k5

__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ void fma2(unsigned long long& acc, unsigned long long a, unsigned long long b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
// All threads of all CTAs of the cluster; orders shared-memory accesses (remote ones included) before and after it.
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Stores 16 bytes at the place of `local` in the shared memory of CTA `cta` of the cluster.
__device__ __forceinline__ void store_cluster_f4(const float* local, uint32_t cta, float a, float b, float c, float d) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(cta));
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// WARPS_M x WARPS_N warps (four in all), each on a 64 x (16 NV) warp tile; NV = 16-byte B vectors
// per lane per k.  <2, 2, 4>: the 128 x 128 tile.  <1, 4, 2>: a 64 x 128 tile of 64 x 32 warp
// tiles (8 x 8 outputs per lane, three CTAs per SM) and <1, 4, 1>: a 64 x 64 tile of 64 x 16 warp
// tiles (8 x 4 outputs per lane, five CTAs per SM) for problems with few tiles.
//
// KSPLIT (64-row tiles only): the kernel is launched in clusters of S = 2 or 4 CTAs that share one output tile; CTA s
// of a cluster multiplies the s-th of S equal ranges of K.  The partial tiles are then added through distributed
// shared memory: the operand buffers, free after the main loop, become S slabs of 64 / S rows; every CTA stores its
// partial of row slab r into slab [its own s] of CTA r (st.shared::cluster), and after a cluster barrier CTA r adds its
// S slabs in the order s = 0, 1, ... and writes alpha * sum + beta * C for its rows.  No workspace, no flags, and the
// order of the additions is fixed, so the result does not depend on timing; it differs from the unsplit forms' in
// rounding (each range is summed on its own first).
template <bool PACKED, int WARPS_M, int WARPS_N, int NV, bool KSPLIT = false>
__global__ void __launch_bounds__(k5::THREADS, NV == 4 ? 2 : (NV == 2 ? 3 : 5))
my_sgemm_kernel_5(int M, int N, int K, float alpha, float* A, float* B, float beta, float* C, int num_blocks_N) {
    using namespace k5;
    static_assert(WARPS_M * WARPS_N == WARPS, "four warps");
    static_assert(!KSPLIT || WARPS_M == 1, "the k-split forms have 64-row tiles");
    constexpr int BM = 64 * WARPS_M;          // rows of the CTA tile (shadows k5::BM)
    constexpr int WN = 16 * NV;               // columns of a warp tile
    constexpr int TILE_N = WARPS_N * WN;      // columns of the CTA tile
    constexpr int A_STRIDE = BM + 4;          // floats between consecutive k in the transposed A slice
    constexpr int A_CH = BM * BK / 4 / THREADS;      // 16-byte chunks of A per thread per slice (4 or 2)
    constexpr int B_CH = BK * TILE_N / 4 / THREADS;  // 16-byte chunks of B per thread per slice (4)
    constexpr int A_FLOATS = 2 * BK * A_STRIDE, B_FLOATS = 2 * BK * TILE_N;
    constexpr int POOL = (KSPLIT && BM * TILE_N > A_FLOATS + B_FLOATS) ? BM * TILE_N : A_FLOATS + B_FLOATS;
    __shared__ __align__(16) float pool[POOL];
    float (*As)[BK * A_STRIDE] = reinterpret_cast<float (*)[BK * A_STRIDE]>(pool);
    float (*Bs)[BK * TILE_N] = reinterpret_cast<float (*)[BK * TILE_N]>(pool + A_FLOATS);

    const int slices = KSPLIT ? static_cast<int>(cluster_size()) : 1;
    const int slice = KSPLIT ? static_cast<int>(cluster_rank()) : 0;
    const int tile = static_cast<int>(blockIdx.x) / slices;
    const int row0 = (tile / num_blocks_N) * BM;
    const int col0 = (tile % num_blocks_N) * TILE_N;
    const int k_begin = slice * (K / slices), k_end = k_begin + K / slices;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tm = lane & 7;
    const int tn = lane >> 3;
    const int wm0 = (warp / WARPS_N) * 64;
    const int wn0 = (warp % WARPS_N) * WN;

    // Chunk c of the A slice: row c / 4, k offset 4 (c % 4): four lanes read one row's 64 bytes.
    float4 pa[A_CH];
    auto load_a = [&](int k0) {
#pragma unroll
        for (int n = 0; n < A_CH; ++n) {
            const int c = threadIdx.x + n * THREADS;
            pa[n] = *reinterpret_cast<const float4*>(A + static_cast<size_t>(row0 + c / (BK / 4)) * K + k0 +
                                                     (c % (BK / 4)) * 4);
        }
    };
    auto store_a = [&](int buf) {
#pragma unroll
        for (int n = 0; n < A_CH; ++n) {
            const int c = threadIdx.x + n * THREADS;
            float* d = &As[buf][(c % (BK / 4)) * 4 * A_STRIDE + c / (BK / 4)];
            d[0] = pa[n].x;
            d[A_STRIDE] = pa[n].y;
            d[2 * A_STRIDE] = pa[n].z;
            d[3 * A_STRIDE] = pa[n].w;
        }
    };
    auto copy_b = [&](int k0, int buf) {
#pragma unroll
        for (int n = 0; n < B_CH; ++n) {
            const int c = threadIdx.x + n * THREADS;
            const int r = c / (TILE_N / 4), c4 = c % (TILE_N / 4);
            cp_async16(&Bs[buf][r * TILE_N + c4 * 4], B + static_cast<size_t>(k0 + r) * N + col0 + c4 * 4);
        }
        cp_async_commit();
    };

    unsigned long long acc2[PACKED ? 8 : 1][PACKED ? 2 * NV : 1];
    float acc[PACKED ? 1 : 8][PACKED ? 1 : 4 * NV];
    if constexpr (PACKED) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 2 * NV; ++j) acc2[i][j] = 0ull;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4 * NV; ++j) acc[i][j] = 0.f;
    }

    load_a(k_begin);
    copy_b(k_begin, 0);
    store_a(0);
    cp_async_wait_all();
    __syncthreads();

    int buf = 0;
    for (int k0 = k_begin; k0 < k_end; k0 += BK) {
        // The other buffer was last read before the barrier that ended the previous slice.
        const bool more = k0 + BK < k_end;
        if (more) {
            load_a(k0 + BK);
            copy_b(k0 + BK, buf ^ 1);
        }
        const float* a_base = &As[buf][wm0 + tm * 4];
        const float* b_base = &Bs[buf][wn0 + tn * 4];
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 alo = *reinterpret_cast<const float4*>(a_base + k * A_STRIDE);
            const float4 ahi = *reinterpret_cast<const float4*>(a_base + k * A_STRIDE + 32);
            const float av[8] = {alo.x, alo.y, alo.z, alo.w, ahi.x, ahi.y, ahi.z, ahi.w};
            if constexpr (PACKED) {
                ulonglong2 b[NV];
#pragma unroll
                for (int j = 0; j < NV; ++j) b[j] = *reinterpret_cast<const ulonglong2*>(b_base + k * TILE_N + j * 16);
                unsigned long long a2[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) a2[i] = pack2(av[i], av[i]);
#pragma unroll
                for (int j = 0; j < NV; ++j) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) fma2(acc2[i][2 * j + 0], a2[i], b[j].x);
#pragma unroll
                    for (int i = 0; i < 8; ++i) fma2(acc2[i][2 * j + 1], a2[i], b[j].y);
                }
            } else {
                float4 b[NV];
#pragma unroll
                for (int j = 0; j < NV; ++j) b[j] = *reinterpret_cast<const float4*>(b_base + k * TILE_N + j * 16);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
#pragma unroll
                    for (int j = 0; j < NV; ++j) {
                        acc[i][4 * j + 0] = fmaf(av[i], b[j].x, acc[i][4 * j + 0]);
                        acc[i][4 * j + 1] = fmaf(av[i], b[j].y, acc[i][4 * j + 1]);
                        acc[i][4 * j + 2] = fmaf(av[i], b[j].z, acc[i][4 * j + 2]);
                        acc[i][4 * j + 3] = fmaf(av[i], b[j].w, acc[i][4 * j + 3]);
                    }
                }
            }
        }
        if (more) store_a(buf ^ 1);
        cp_async_wait_all();
        __syncthreads();
        buf ^= 1;
    }

    if constexpr (KSPLIT) {
        // This CTA finishes row slab `slice` of the tile: slab_rows x TILE_N outputs, MAX_OUT 16-byte pieces per
        // thread at most (S = 2).  Their old values of C are fetched now, so that the loads are in flight while the
        // partial sums travel.
        constexpr int MAX_OUT = (BM / 2) * (TILE_N / 4) / THREADS;
        const int slab_shift = 6 - (slices >> 1);          // 64 / S rows per slab, S = 2 or 4
        const int slab_rows = 1 << slab_shift;
        const int outs = slab_rows * (TILE_N / 4);
        float4 old[MAX_OUT];
#pragma unroll
        for (int n = 0; n < MAX_OUT; ++n) {
            const int e = threadIdx.x + n * THREADS;
            if (e < outs)
                old[n] = *reinterpret_cast<const float4*>(C + static_cast<size_t>(row0 + slice * slab_rows + e / (TILE_N / 4)) * N +
                                                          col0 + (e % (TILE_N / 4)) * 4);
        }
        // Every CTA of the cluster is past its main loop (its pool is free) before anyone stores into it.
        cluster_barrier();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = i < 4 ? tm * 4 + i : 32 + tm * 4 + (i - 4);
            const float* slot = pool + ((slice << slab_shift) + (r & (slab_rows - 1))) * TILE_N + wn0 + tn * 4;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                float r0, r1, r2, r3;
                if constexpr (PACKED) {
                    unpack2(acc2[i][2 * j + 0], r0, r1);
                    unpack2(acc2[i][2 * j + 1], r2, r3);
                } else {
                    r0 = acc[i][4 * j + 0]; r1 = acc[i][4 * j + 1]; r2 = acc[i][4 * j + 2]; r3 = acc[i][4 * j + 3];
                }
                store_cluster_f4(slot + j * 16, static_cast<uint32_t>(r >> slab_shift), r0, r1, r2, r3);
            }
        }
        cluster_barrier();
        // S partial slabs of slab_rows x TILE_N, added in the order of the k ranges.
#pragma unroll
        for (int n = 0; n < MAX_OUT; ++n) {
            const int e = threadIdx.x + n * THREADS;
            if (e < outs) {
                const int lr = e / (TILE_N / 4), c4 = e % (TILE_N / 4);
                float4 sum = *reinterpret_cast<const float4*>(pool + lr * TILE_N + c4 * 4);
                for (int sl = 1; sl < slices; ++sl) {
                    const float4 p = *reinterpret_cast<const float4*>(pool + ((sl << slab_shift) + lr) * TILE_N + c4 * 4);
                    sum.x += p.x; sum.y += p.y; sum.z += p.z; sum.w += p.w;
                }
                float4 v = old[n];
                v.x = alpha * sum.x + beta * v.x;
                v.y = alpha * sum.y + beta * v.y;
                v.z = alpha * sum.z + beta * v.z;
                v.w = alpha * sum.w + beta * v.w;
                *reinterpret_cast<float4*>(C + static_cast<size_t>(row0 + slice * slab_rows + lr) * N + col0 + c4 * 4) = v;
            }
        }
        return;
    }

    // C = alpha * acc + beta * C, 16 bytes at a time.
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = row0 + wm0 + (i < 4 ? tm * 4 + i : 32 + tm * 4 + (i - 4));
        float* c_row = C + static_cast<size_t>(r) * N + col0 + wn0 + tn * 4;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            float4* c = reinterpret_cast<float4*>(c_row + j * 16);
            float4 v = *c;
            float r0, r1, r2, r3;
            if constexpr (PACKED) {
                unpack2(acc2[i][2 * j + 0], r0, r1);
                unpack2(acc2[i][2 * j + 1], r2, r3);
            } else {
                r0 = acc[i][4 * j + 0]; r1 = acc[i][4 * j + 1]; r2 = acc[i][4 * j + 2]; r3 = acc[i][4 * j + 3];
            }
            v.x = alpha * r0 + beta * v.x;
            v.y = alpha * r1 + beta * v.y;
            v.z = alpha * r2 + beta * v.z;
            v.w = alpha * r3 + beta * v.w;
            *c = v;
        }
    }
}

namespace {

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

std::mutex g_sgemm_mu;   // guards the caches below; entry points may be called from several host threads

int sm_count() {
    static int n[64] = {};
    std::lock_guard<std::mutex> lk(g_sgemm_mu);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (n[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        n[dev] = v;
    }
    return n[dev];
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Bounds-checked tiled kernel: any shape.
int launch_generic(int M, int N, int K, float alpha, const float* A, const float* B, float beta, float* C,
                   cudaStream_t s) {
    constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
    const int nbn = ceil_div(N, BN);
    const long long blocks = static_cast<long long>(ceil_div(M, BM)) * nbn;
    if (blocks > 0x7fffffffLL) return set_error(PRISM_B200_ERR_TOO_LARGE, "sgemm: too many tiles");
    my_sgemm_kernel_3<BM, BN, BK, TM, TN>
        <<<static_cast<unsigned>(blocks), (BM * BN) / (TM * TN), 0, s>>>(M, N, K, alpha, A, B, beta, C, nbn);
    return PRISM_B200_OK;
}

bool g_k5_scalar = false;  // PRISM_B200_SGEMM_SCALAR=1 selects the plain fmaf form of kernel 5 (same bits, slower)
bool g_k5_env_read = false;
int g_k5_tile_mode = -1;   // prism_b200_sgemm_tile_mode: -1 = by shape, 0 / 1 / 2 = 128 x 128 / 64 x 128 / 64 x 64 (tests)
int g_k5_slices = -1;      // prism_b200_sgemm_k_slices: -1 = by shape, 1 / 2 / 4 = CTAs that share a tile along K (tests)

// Kernel 5's tile (0: 128 x 128, 1: 64 x 128, 2: 64 x 64) and the CTAs per tile along K (1, 2 or 4; the 64-row tiles
// only) for an M x N x K problem that the tiled forms divide, on a device with `sms` SMs: the candidate with the
// shortest estimated makespan.  want_form >= 0 restricts the tile; want_slices > 0 fixes the sharing (halved until
// K divides into 16-wide steps per CTA).
void k5_plan(int M, int N, int K, int sms, int want_form, int want_slices, int* form, int* slices) {
    double best = -1.0;
    for (int f = 0; f < 3; ++f) {
        if (want_form >= 0 && f != want_form) continue;
        const long long ctas = static_cast<long long>(M / (f == 0 ? 128 : 64)) * (N / (f == 2 ? 64 : 128));
        const double per_step = f == 0 ? 2.0 / 1.043 : (f == 1 ? 1.0 : 0.5 / 0.75);
        const int most = f == 0 ? 1 : 4;
        int fixed = 0;
        if (want_slices > 0) {
            fixed = want_slices < most ? want_slices : most;
            while (fixed > 1 && K % (k5::BK * fixed) != 0) fixed >>= 1;
        }
        for (int sl = 1; sl <= most; sl *= 2) {
            if (fixed ? sl != fixed : K % (k5::BK * sl) != 0) continue;
            const long long rounds = (ctas * sl + sms - 1) / sms;
            // one four-warp CTA alone on an SM cannot hide its own latencies; two hide most of them
            const double alone = f == 0 ? (rounds >= 2 ? 1.0 : 0.9) : (rounds >= 3 ? 1.0 : (rounds == 2 ? 0.95 : 0.88));
            const double cost = static_cast<double>(rounds) * (static_cast<double>(K / sl) + (sl == 1 ? 32.0 : 48.0)) * per_step / alone;
            if (best < 0.0 || cost < best) {
                best = cost;
                *form = f;
                *slices = sl;
            }
        }
    }
}

}  // namespace
}  // namespace prism_b200

using namespace prism_b200;

extern "C" int prism_b200_sgemm_tile_mode(int mode) {
    if (mode < -1 || mode > 2) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "sgemm_tile_mode: -1, 0, 1 or 2");
    std::lock_guard<std::mutex> lk(g_sgemm_mu);
    g_k5_tile_mode = mode;
    return PRISM_B200_OK;
}

extern "C" int prism_b200_sgemm_k_slices(int slices) {
    if (slices != -1 && slices != 1 && slices != 2 && slices != 4)
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "sgemm_k_slices: -1, 1, 2 or 4");
    std::lock_guard<std::mutex> lk(g_sgemm_mu);
    g_k5_slices = slices;
    return PRISM_B200_OK;
}

extern "C" int prism_b200_sgemm_plan(int M, int N, int K, int sms, int* tile, int* slices) {
    if (!tile || !slices || M <= 0 || N <= 0 || K <= 0 || sms < 1)
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "sgemm_plan: bad argument");
    if (M % k5::BM || N % k5::BN || K % k5::BK) {
        *tile = -1;      // no tiled form divides this shape: the bounds-checked kernel runs
        *slices = 1;
        return PRISM_B200_OK;
    }
    int want_form, want_slices;
    {
        std::lock_guard<std::mutex> lk(g_sgemm_mu);
        want_form = g_k5_tile_mode;
        want_slices = g_k5_slices;
    }
    k5_plan(M, N, K, sms, want_form, want_slices, tile, slices);
    return PRISM_B200_OK;
}

extern "C" int prism_b200_sgemm(int kernel_id, int M, int N, int K, float alpha, const float* A, const float* B,
                                float beta, float* C, void* stream) {
    if (kernel_id < 1 || kernel_id > 6)
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "sgemm: unknown kernel id %d (1..6)", kernel_id);
    if (M < 0 || N < 0 || K < 0) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "sgemm: negative dimension");
    if (M == 0 || N == 0) return PRISM_B200_OK;
    if (!C || (K > 0 && (!A || !B))) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "sgemm: null pointer");
    if (static_cast<long long>(M) * N > 0x7fffffffLL * 256LL)
        return set_error(PRISM_B200_ERR_TOO_LARGE, "sgemm: M*N too large");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (int rc = bind_status_word()) return rc;
    const bool vec_ok = aligned16(A) && aligned16(B) && aligned16(C);
    int rc = PRISM_B200_OK;

    switch (kernel_id) {
    case 1: {
        const int block = 256;
        const long long blocks = (static_cast<long long>(M) * N + block - 1) / block;
        my_sgemm_kernel_1<<<static_cast<unsigned>(blocks), block, 0, s>>>(M, N, K, alpha, A, B, beta, C, block);
        break;
    }
    case 2: {
        const int tile = 32;
        const long long blocks = static_cast<long long>(ceil_div(M, tile)) * ceil_div(N, tile);
        my_sgemm_kernel_2<<<static_cast<unsigned>(blocks), tile * tile, 0, s>>>(M, N, K, alpha, A, B, beta, C, tile);
        break;
    }
    case 3: {
        constexpr int BS = 32;
        if (M % BS == 0 && N % BS == 0 && K % BS == 0 && K > 0) {
            const int nbn = N / BS;
            sgemm_shared_mem_block<BS><<<(M / BS) * nbn, BS * BS, 0, s>>>(M, N, K, alpha, A, B, beta, C, nbn);
        } else {
            rc = launch_generic(M, N, K, alpha, A, B, beta, C, s);
        }
        break;
    }
    case 4: {
        if (M % 128 == 0 && N % 128 == 0 && K % 8 == 0 && K > 0 && vec_ok) {
            const int nbn = N / 128;
            my_sgemm_kernel_4<128, 128, 8, 8, 8><<<(M / 128) * nbn, 256, 0, s>>>(
                M, N, K, alpha, const_cast<float*>(A), const_cast<float*>(B), beta, C, nbn);
        } else {
            rc = launch_generic(M, N, K, alpha, A, B, beta, C, s);
        }
        break;
    }
    case 5: {
        if (M % k5::BM == 0 && N % k5::BN == 0 && K % k5::BK == 0 && K > 0 && vec_ok) {
            int want_form, want_slices;
            {
                std::lock_guard<std::mutex> lk(g_sgemm_mu);
                if (!g_k5_env_read) {
                    const char* e = getenv("PRISM_B200_SGEMM_SCALAR");
                    g_k5_scalar = e && e[0] == '1';
                    g_k5_env_read = true;
                }
                want_form = g_k5_tile_mode;
                want_slices = g_k5_slices;
            }
            // Which tile (0: 128 x 128, 1: 64 x 128, 2: 64 x 64) and how many CTAs per tile along K (1, 2 or 4; the 64-row
            // tiles only): the candidate with the shortest estimated makespan.  An SM works through ceil(CTAs / SMs) CTAs
            // of K / S k-steps each (plus a fixed start-up and write-out cost, larger where partial tiles are exchanged), at
            // a cost per k-step that follows the tile's area and its measured rate at 4096^3 (62.4 / 59.8 / 45.0 TFLOP/s),
            // raised where an SM holds only one or two CTAs at a time.
            // On a B200 this estimate ranks the candidates as measured within a few per cent from 512^3 to 4096^3 and
            // for 512 ... 2048 x 4096 x 4096: e.g. 1280^3 36.3 -> 46.2 TFLOP/s and 2048^3 51.6 -> 56.5 with 64 x 128
            // tiles shared by two CTAs (7 rounds of half-length CTAs instead of 2 rounds of 128 x 128 ones), 512^3
            // 11.5 -> 18.8 shared by four.  The unshared forms add one element's products in the same k order and give
            // the same bits; a shared tile sums each range of K first.
            int form = 0, slices = 1;
            k5_plan(M, N, K, sm_count(), want_form, want_slices, &form, &slices);
            void (*kern)(int, int, int, float, float*, float*, float, float*, int) =
                form == 2   ? (g_k5_scalar ? my_sgemm_kernel_5<false, 1, 4, 1> : my_sgemm_kernel_5<true, 1, 4, 1>)
                : form == 1 ? (g_k5_scalar ? my_sgemm_kernel_5<false, 1, 4, 2> : my_sgemm_kernel_5<true, 1, 4, 2>)
                            : (g_k5_scalar ? my_sgemm_kernel_5<false, 2, 2, 4> : my_sgemm_kernel_5<true, 2, 2, 4>);
            const int tile_n = form == 2 ? 64 : 128;
            const int nbn = N / tile_n;
            const long long blocks = static_cast<long long>(M / (form == 0 ? 128 : 64)) * nbn;
            if (slices > 1) {
                kern = form == 2 ? (g_k5_scalar ? my_sgemm_kernel_5<false, 1, 4, 1, true> : my_sgemm_kernel_5<true, 1, 4, 1, true>)
                                 : (g_k5_scalar ? my_sgemm_kernel_5<false, 1, 4, 2, true> : my_sgemm_kernel_5<true, 1, 4, 2, true>);
                cudaLaunchConfig_t cfg{};
                cudaLaunchAttribute attr[1];
                cfg.gridDim = dim3(static_cast<unsigned>(blocks * slices));
                cfg.blockDim = dim3(k5::THREADS);
                cfg.stream = s;
                attr[0].id = cudaLaunchAttributeClusterDimension;
                attr[0].val.clusterDim.x = static_cast<unsigned>(slices);
                attr[0].val.clusterDim.y = 1;
                attr[0].val.clusterDim.z = 1;
                cfg.attrs = attr;
                cfg.numAttrs = 1;
                PRISM_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, M, N, K, alpha, const_cast<float*>(A), const_cast<float*>(B), beta, C,
                                                  nbn));
            } else {
                kern<<<static_cast<unsigned>(blocks), k5::THREADS, 0, s>>>(
                    M, N, K, alpha, const_cast<float*>(A), const_cast<float*>(B), beta, C, nbn);
            }
        } else {
            rc = launch_generic(M, N, K, alpha, A, B, beta, C, s);
        }
        break;
    }
    case 6:
        rc = launch_generic(M, N, K, alpha, A, B, beta, C, s);
        break;
    }
    if (rc) return rc;
    PRISM_CUDA_TRY(cudaGetLastError());
    count_launch();
    return PRISM_B200_OK;
}
