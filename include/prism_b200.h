/*
 * prism_b200 -- C ABI of the B200 (sm_100a) kernels that stand in for the
 * three kernel families of the Prism evaluation harnesses.
 *
 * Every entry point is `extern "C"`, takes plain device pointers and sizes,
 * enqueues its work on the given CUDA stream and returns immediately with a
 * status code (0 = PRISM_B200_OK).  Nothing here calls exit()/abort(); no
 * device code traps.  Device-side waits are bounded: a wait that runs out
 * writes a code into a status word that prism_b200_last_error() reports after
 * the stream has been synchronised.
 *
 * Ownership: the caller allocates and frees every device buffer, including
 * the scan workspace.  The library owns only cached TMA tensor maps and one
 * pinned status word per process.
 *
 * `stream` is a cudaStream_t passed as void* so that this header needs no
 * CUDA include (NULL = the legacy default stream).
 */
#ifndef PRISM_B200_H
#define PRISM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes -------------------------------------------------------- */
enum {
    PRISM_B200_OK = 0,
    PRISM_B200_ERR_INVALID_ARGUMENT = 1, /* null pointer, negative size, bad kernel id   */
    PRISM_B200_ERR_UNSUPPORTED_SHAPE = 2,/* shape outside what the chosen kernel accepts  */
    PRISM_B200_ERR_MISALIGNED = 3,       /* pointer not aligned for 16-byte accesses      */
    PRISM_B200_ERR_CUDA = 4,             /* a CUDA runtime/driver call failed             */
    PRISM_B200_ERR_DEVICE_TIMEOUT = 5,   /* a bounded device-side wait ran out            */
    PRISM_B200_ERR_TOO_LARGE = 6         /* size beyond a stated maximum                  */
};

/* ---- library ------------------------------------------------------------- */

/* Version as major*10000 + minor*100 + patch. */
int prism_b200_version(void);

/*
 * Last error seen by this process.  `code` receives the most recent non-zero
 * status returned by an entry point or raised by a kernel (device-side
 * timeouts become visible once the stream is synchronised); `msg` receives a
 * short text.  Returns the same code.  Either pointer may be NULL.
 * Replaces the reference's `cudaCheck` -> `exit(EXIT_FAILURE)` policy
 * (evals/4090_sgemm/runner.cu:16-22, evals/4090_scan/scan_harness.cuh:15-25).
 */
int prism_b200_last_error(int* code, char* msg, size_t len);

/* Clears the sticky error state (host side and the device status word). */
void prism_b200_clear_error(void);

/*
 * Exercises the device-side error path without any fault: one warp waits at most limit_ns
 * (1 ns .. 10 ms) for a barrier that nothing completes, records the timeout and returns.  After the
 * stream is synchronised prism_b200_last_error() reports PRISM_B200_ERR_DEVICE_TIMEOUT; the context
 * stays usable.  The reference has no device-side error path (its waits spin without bound,
 * generated/lookback_to_prev_blocks.cu:13-14, evals/h100_bench/utils.cuh:259-273).
 */
int prism_b200_selftest_wait_timeout(unsigned long long limit_ns, void* stream);

/* Number of kernels this library has launched since load (all entry points). */
unsigned long long prism_b200_launch_count(void);

/* ---- FP32 SGEMM: C = alpha * A * B + beta * C ----------------------------- */

/*
 * Replaces `run_my_kernel(int my_kernel_num, M, N, K, alpha, A, B, beta, C)`
 * (evals/4090_sgemm/runner.cu:245-267, declared in runner.cuh:28-29).
 * A is M x K, B is K x N, C is M x N, all row-major fp32 in device memory, C is
 * updated in place.  kernel_id follows the evaluation harness:
 *   1  one thread per C element              (generated/my_sgemm_kernel_1.cu)
 *   2  32x32-tile thread remap, coalesced    (generated/my_sgemm_kernel_2.cu)
 *   3  32x32 shared-memory tiles             (generated/sgemm_shared_mem_block.cu,
 *                                             which evals/run_4090.sh:67-69 renames to kernel 3)
 *   4  128x128x8 tiles, 8x8 register tile, 128-bit accesses
 *                                            (generated/my_sgemm_kernel_4.cu)
 *   5  warp-tiled 128x128 tile, 8x16 accumulators per thread; on B200 A is
 *      transposed into shared memory, B arrives by cp.async, and the FMAs are
 *      issued two at a time as fma.rn.f32x2
 *                                            (generated/my_sgemm_kernel_5.cu)
 *   6  register-tiled, scalar accesses       (generated/my_sgemm_kernel_3.cu,
 *                                             emitted by the reference but never launched by its harness)
 * Shapes: ids 1, 2 and 6 accept any positive M, N, K.  Ids 3, 4, 5 use their tiled
 * kernels when the shape divides the tile (3: multiples of 32; 4: M, N multiples of
 * 128, K of 8; 5: M, N multiples of 128, K of 16) and a bounds-checked tiled kernel
 * otherwise, so no shape is rejected and no shape reads out of bounds.
 * No TF32 and no tensor cores anywhere on this path.
 */
int prism_b200_sgemm(int kernel_id, int M, int N, int K, float alpha,
                     const float* A, const float* B, float beta, float* C,
                     void* stream);

/*
 * Tile of kernel 5: -1 (default) the launcher picks among 128 x 128, 64 x 128 and 64 x 64 (and, for the 64-row tiles,
 * how many CTAs share a tile along K, below) by an estimate of the makespan: rounds of CTAs per SM x k-steps per CTA x
 * the tile's cost per step; 0 / 1 / 2 forces 128 x 128 / 64 x 128 / 64 x 64.  The three tiles give the same bits.
 * Process-wide; for tests and measurements.  The reference's launcher has one tile per kernel
 * (evals/4090_sgemm/runner.cu:191-243).
 */
int prism_b200_sgemm_tile_mode(int mode);

/*
 * CTAs of kernel 5 that share one output tile along K: -1 (default) the launcher picks (1; 2 or 4 where the 64-row
 * tiles still leave the SMs mostly without a second CTA and K is long enough), 1 / 2 / 4 forces it for the 64 x 128 and
 * 64 x 64 tiles (halved until K divides into 16-wide steps per CTA; 128 x 128 tiles are never shared).  The S CTAs of a
 * tile form a thread-block cluster, multiply one range of K each and add the partial tiles through distributed shared
 * memory in the order of the ranges, so the result is the same on every run; it differs from the unshared forms' in
 * rounding only (<= 1e-5 relative to fp64 like them).  Process-wide; for tests and measurements.  The reference has
 * no k-split (evals/4090_sgemm/runner.cu:191-243).
 */
int prism_b200_sgemm_k_slices(int slices);

/*
 * What the launcher of kernel 5 would take for an M x N x K problem on a device with `sms` SMs, under the two switches
 * above: *tile = 0 / 1 / 2 (128 x 128 / 64 x 128 / 64 x 64) and *slices = 1 / 2 / 4, or *tile = -1 where no tiled form
 * divides the shape (M, N multiples of 128 and K of 16 are needed) and the bounds-checked kernel runs.  Host-side
 * arithmetic only (no GPU needed); the estimate is rounds of CTAs per SM x (K / slices + a fixed cost) x the tile's cost
 * per k-step, raised where an SM holds only one or two CTAs.  No counterpart in the reference.
 */
int prism_b200_sgemm_plan(int M, int N, int K, int sms, int* tile, int* slices);

/* ---- uint32 inclusive scan (single pass, decoupled look-back) ------------- */

/*
 * Replaces `get_workspace_size(n)` (evals/4090_scan/main.cu:63-66).
 * Bytes of device scratch prism_b200_scan needs for n elements.
 */
int prism_b200_scan_workspace_size(size_t n, size_t* bytes);

/*
 * Replaces `launch_scan(n, x, workspace)` (evals/4090_scan/main.cu:68-86).
 * In-place inclusive prefix sum of n uint32 (wrap-around adds, bit-identical to
 * int32).  Any n >= 0 is accepted (the reference needs n % 16384 == 0); n must
 * be below 2^32.  x must be 16-byte aligned.  The workspace may hold anything on
 * entry: it is re-armed on the stream before the kernel, as the reference does.
 */
int prism_b200_scan(size_t n, uint32_t* x, void* workspace, void* stream);

/*
 * fp32 flavour of the same single-pass kernel (no counterpart in the reference, whose scan is
 * uint32 only): in-place inclusive prefix sum of n floats, same workspace, same limits.  Sums
 * are formed in fp32, 4 elements serially per thread, then by warp shuffles, then across tiles
 * through the look-back; how the tile sums are grouped follows the look-back windows, which
 * depend on timing, so two runs may differ in the last bits (compare with a tolerance).
 */
int prism_b200_scan_f32(size_t n, float* x, void* workspace, void* stream);

/*
 * The other flavours of the same kernel (no counterpart in the reference): separate input and
 * output (in == out is allowed, partial overlap is not), inclusive or exclusive, and the element type:
 * uint32 (default), fp32 adds (PRISM_B200_SCAN_F32) or 64-bit integers with wrap-around adds
 * (PRISM_B200_SCAN_I64, bit-identical for int64 and uint64; n counts elements, in and out hold 8 n bytes).
 * Exclusive: out[0] = 0, out[i] = in[0] + ... + in[i-1].  Limits and alignment as for prism_b200_scan;
 * flags = 0 with in == out is prism_b200_scan.  The 64-bit flavour needs twice the records per element
 * (its tiles hold 2048 elements): size its workspace with prism_b200_scan_general_workspace_size, which
 * for the 32-bit flavours returns what prism_b200_scan_workspace_size returns.
 */
#define PRISM_B200_SCAN_EXCLUSIVE 1
#define PRISM_B200_SCAN_F32 2
#define PRISM_B200_SCAN_I64 4
int prism_b200_scan_general(size_t n, const void* in, void* out, void* workspace, int flags, void* stream);
int prism_b200_scan_general_workspace_size(size_t n, int flags, size_t* bytes);

/*
 * Sharded scan helpers (no counterpart in the reference, which is single-GPU).
 * A rank that owns the r-th contiguous chunk of a longer array
 *   1. prism_b200_reduce_u32: total of its chunk -> *total (device),
 *   2. exchanges totals with the other ranks (an all-gather of one word each),
 *   3. prism_b200_scan_seeded: scans its chunk starting from
 *      totals[0] + ... + totals[rank-1] (read on the device, wrap-around adds).
 * prism_b200_scan_add_carry adds the same carry to an already scanned chunk
 * (the two-pass form: local scan, exchange, carry add).
 */
int prism_b200_reduce_u32(size_t n, const uint32_t* x, uint32_t* total, void* stream);
int prism_b200_scan_seeded(size_t n, uint32_t* x, void* workspace,
                           const uint32_t* totals, int rank, void* stream);
int prism_b200_scan_add_carry(size_t n, uint32_t* x, const uint32_t* totals,
                              int rank, void* stream);

/*
 * The same exchange without a collective call, over peer memory (NVLink / NVSwitch).  Every rank
 * owns an array `slots` of 2 * world 64-bit words that all ranks can write (peer-mapped or
 * symmetric memory, zeroed once); `peer_slots` is a device array of the `world` base addresses of
 * these arrays, in rank order.  `epoch` is non-zero, the same on every rank, and changes from call
 * to call (1, 2, 3, ...).
 *
 * prism_b200_scan_sharded does the whole step in ONE launch.  phases = 3:
 *   reduce   the CTAs add up the chunk slice by slice (last slice first, so that the start of the
 *            chunk is what remains in L2); whoever finishes the last slice stores {epoch, total}
 *            into slot (epoch & 1) * world + rank of EVERY rank's array, one 64-bit store each;
 *   scan     the chunk is scanned in place; its first tile waits until all `world` words of this
 *            epoch have arrived in this rank's own array and starts from the sum of the lower
 *            ranks' totals.
 * phases = 1 or 2 runs one of the two alone (a reduce-only launch on every rank, then a scan-only
 * launch on every rank, is the same computation in two launches).
 * The wait for the words is bounded by wait_limit_ns (0 = 1 s, at most 600 s): ranks that enter the
 * call further apart than that give up, set PRISM_B200_ERR_DEVICE_TIMEOUT (see prism_b200_last_error,
 * after synchronising) and leave x undefined, where a collective would have waited.  Pick the limit
 * for the skew the job can have.  An empty chunk (n = 0) still publishes a zero total and waits.
 * Waiting for every rank's word, together with the two alternating halves of the array, is what
 * makes it safe for a rank to run a whole call ahead of another.  world <= 32.
 * With phases = 2, rank may equal world: the piece then lies behind every rank's chunk and starts from the sum of
 * ALL totals.  That is what lets one rank own a head and a tail of the array (prism_b200/sharded.py, the
 * "head_tail" schedule): it scans the head outright (its prefix is zero), publishes the head's total with
 * prism_b200_scan_publish_total while the others are still adding up their chunks, and scans the tail, whose total
 * nobody needs, once all words are in -- 8 bytes per element on that rank instead of 12, so it can own 1.5 chunks
 * and the whole array finishes in the time of world + 0.5 chunks' worth of 12-byte traffic instead of world.
 * The pieces are also exported on their own: prism_b200_scan_publish_total stores the word for a
 * total computed elsewhere (prism_b200_reduce_u32), prism_b200_scan_seeded_peers is phases = 2
 * with the default limit.  No counterpart in the reference.
 */
#define PRISM_B200_SHARD_REDUCE 1
#define PRISM_B200_SHARD_SCAN 2
int prism_b200_scan_sharded(size_t n, uint32_t* x, void* workspace, const uint64_t* slots,
                            uint64_t* const* peer_slots, int rank, int world, uint32_t epoch, int phases,
                            unsigned long long wait_limit_ns, void* stream);
int prism_b200_scan_publish_total(const uint32_t* total, uint64_t* const* peer_slots, int world,
                                  int rank, uint32_t epoch, void* stream);
int prism_b200_scan_seeded_peers(size_t n, uint32_t* x, void* workspace, const uint64_t* slots,
                                 int rank, int world, uint32_t epoch, void* stream);

/*
 * Scan without caller-provided scratch and without any allocation.  No
 * counterpart in the reference (its launcher always takes a workspace,
 * evals/4090_scan/main.cu:68-86).
 *
 * For callers that cannot allocate device memory where the scan runs: plugins
 * that only ever see buffers owned by their host application, loops that may
 * not block on the allocator, processes whose device memory is already all
 * handed out.  Same result as prism_b200_scan, in place, but the look-back
 * records live in a fixed 2,097,280-byte array inside the library's device image
 * (every GPU that loads the library holds it until exit), which bounds n:
 *   n <= 2^28 elements; larger n returns PRISM_B200_ERR_TOO_LARGE.
 * The call performs no cudaMalloc/cudaFree and calls no allocating routine.
 * The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress) and should therefore come before any stream capture.
 * All calls on a device share the one array and it is re-armed at the start of
 * each call, so two calls whose GPU work overlaps (different streams, or
 * different host threads) race with each other: serialise them.  A device-side
 * timeout is reported through prism_b200_last_error only if another entry point
 * has already set up the status word on that device, since doing so allocates
 * pinned memory, which this entry point will not do.
 */
int prism_b200_scan_static(size_t n, uint32_t* x, void* stream);

/* ---- bf16 GEMM: C = A * B^T, fp32 accumulate ------------------------------ */

/*
 * Replaces `runmyh100(M, N, K, A, B, C, DB)` (evals/h100_bench/utils.cuh:504-533),
 * the launcher of `cutlass_my_h100_match_no_tail`
 * (generated/cutlass_my_h100_match_no_tail.cu:1-370).
 * A is M x K and B is N x K, both K-major (row-major) bf16; C is M x N bf16 stored
 * COLUMN-major, C[n * M + m], as the reference kernel writes it
 * (generated/cutlass_my_h100_match_no_tail.cu:313,347-354).  fp32 accumulation,
 * round-to-nearest-even on store.  Requires M % 128 == 0, N % 128 == 0, K % 64 == 0, K > 0
 * (the reference needs M % 2048 == 0, N % 2048 == 0, K % 256 == 0).
 * Tensor maps are cached on (device, pointer, rows, K) so a new buffer never reuses a
 * stale map (the reference caches on M alone, utils.cuh:512-518).
 * bf16 values are passed as uint16_t bit patterns to keep this header free of CUDA types.
 */
int prism_b200_gemm_bf16(int M, int N, int K, const uint16_t* A, const uint16_t* B,
                         uint16_t* C, void* stream);

/*
 * The same product with a scaling epilogue: D = alpha * (A * B^T) + beta * Cin, all three matrices in the
 * layouts of prism_b200_gemm_bf16 (Cin and D column-major M x N bf16; Cin == D is allowed, partial overlap is
 * not).  The sum alpha * acc + beta * Cin is formed in fp32 from the fp32 accumulator and rounded once; with
 * beta == 0 the values of Cin do not enter (NaN included).  No
 * counterpart in the reference, whose bf16 kernel has no alpha/beta (its SGEMM kernels do,
 * generated/my_sgemm_kernel_5.cu:56-77).  Runs on the one-CTA form of the kernel for every shape.
 */
int prism_b200_gemm_bf16_axpby(int M, int N, int K, float alpha, const uint16_t* A, const uint16_t* B, float beta,
                               const uint16_t* Cin, uint16_t* D, void* stream);

/*
 * How the 512 x 256 two-CTA form of prism_b200_gemm_bf16 deals its output tiles to its CTA pairs.  With `tiles` tiles on
 * `pairs` pairs, a pair computes the whole tiles pair, pair + pairs, ... of the tiles / pairs full waves.  The
 * R = tiles mod pairs tiles that remain would occupy R pairs for a whole tile's time while the others idle; with
 * fill = 1 each of them is cut into its two 256-row blocks of n, which a pair computes on its own over all of K with
 * nothing to hand over (piece q = pair + j * pairs is block q mod 2 of tile (tiles / pairs) * pairs + q / 2), so where
 * 2 R <= pairs the last wave takes half a tile's time.  A piece accumulates its k-blocks in the order a whole tile
 * does, so results are bit-identical with and without the fill.  The launcher fills where that halves the last wave
 * (on a B200's 74 pairs: 8192^3 cut over 2 GPUs, 256 tiles = 3 waves + 34).
 *
 * prism_b200_gemm_bf16_fill_plan writes the items of pair `pair` in the order it computes them, as (tile, block) with
 * block = -1 for a whole tile, into tile_block[0 .. 2 * min(*count, capacity)) and their number into *count.  Host-side
 * arithmetic only (no GPU needed); it is the function the kernel evaluates.  The reference's kernel has a fixed grid of
 * 128 CTAs, one tile each, and nothing like it (generated/cutlass_my_h100_match_no_tail.cu:90-101).
 */
int prism_b200_gemm_bf16_fill_plan(int tiles, int pairs, int fill, int pair, int capacity, int* tile_block, int* count);
/* -1 (default): the launcher decides by shape; 0: never cut the last wave; 2: cut it whenever it is partly filled.
 * Process-wide; overrides the environment variable PRISM_B200_GEMM_FILL.  For tests and measurements. */
int prism_b200_gemm_bf16_fill_mode(int mode);

/* ---- one-sided all-gather over peer memory --------------------------------- */

/*
 * The exchange step of the multi-GPU host-buffer GEMM (no counterpart in the reference, which is single-GPU):
 * every rank pushes its piece of a block into every other rank's buffer over NVLink and raises a flag there; a
 * consumer waits for all ranks' flags before it reads the block from its OWN memory.  All buffers must be
 * peer-mapped (e.g. torch symmetric memory); `peer_dst` / `peer_flags` are device arrays of the `world` base
 * addresses in rank order; `epoch` is non-zero, the same on every rank, and grows by one per call.
 *   prism_b200_peer_push  copies `bytes` (a multiple of 16) from `src` to `dst_offset` in every OTHER rank's buffer
 *                         (this rank's own copy is expected to be in place already), then stores `epoch` into flag
 *                         word `flag_index` of every rank, its own included.  `done_counter` is one zeroed device
 *                         word owned by the caller (the kernel leaves it zero).
 *   prism_b200_peer_wait  waits on the stream until flag words [first, first + count) of this rank's own array hold
 *                         `epoch` or a later one, for at most wait_limit_ns (0 = 1 s); a wait that runs out sets
 *                         PRISM_B200_ERR_DEVICE_TIMEOUT (prism_b200_last_error after synchronising).
 * A rank can be one call ahead of another, so callers alternate between two destination buffers by the parity
 * of the epoch.  world <= 32.
 */
int prism_b200_peer_push(const void* src, size_t bytes, void* const* peer_dst, size_t dst_offset, int world, int rank,
                         uint32_t* const* peer_flags, int flag_index, uint32_t epoch, uint32_t* done_counter,
                         void* stream);
int prism_b200_peer_wait(const uint32_t* flags, int first, int count, uint32_t epoch,
                         unsigned long long wait_limit_ns, void* stream);

/* ---- host-buffer plans ------------------------------------------------------ */

/*
 * The three operators for operands that live in HOST memory, which is how the reference
 * harnesses hold theirs: they cudaMemcpy in, launch, cudaMemcpy out
 * (evals/4090_scan/scan_harness.cuh:112-131, evals/4090_sgemm/main.cu:64-120,
 * evals/h100_bench/main.cu:105-130).  A plan owns device staging buffers for one problem size
 * and three streams; a run cuts the call into blocks that are contiguous on both sides and
 * overlaps the upload of one block, the kernel on the one before and the download of the one
 * before that (bf16 GEMM: A whole, then rows of B = row blocks of the N x M result; SGEMM: B
 * whole, then rows of M of A and C; scan: blocks of the array, each seeded on the device with
 * the last element of the block before).  Host buffers should be pinned (cudaHostAlloc /
 * cudaHostRegister), otherwise the copies do not overlap; results are the same either way and
 * bit-identical to the device-resident entry points (for SGEMM kernel 5: where neither call shares a tile along K, see
 * prism_b200_sgemm_k_slices; otherwise both are within the same bound of fp64 and differ in rounding).
 * A run is asynchronous: it is ordered after the work already queued on `stream`, and `stream`
 * waits for it; synchronise `stream` before reading the host result.  Runs of one plan must
 * not overlap each other except through that ordering.  create/destroy allocate and free
 * device memory, a run does not.  block_rows / block_elems = 0 picks the default (bf16 GEMM: blocks of 1024 rows of B,
 * SGEMM: M / 16 rows of A rounded up to 128; either with the last block cut again in halves down to 256 / 128 rows, so
 * that little is left to do after the last upload; scan: n / 16 elements, at least 2^22).  Operand layouts and dtypes are those of prism_b200_gemm_bf16,
 * prism_b200_sgemm and prism_b200_scan.  A plan belongs to the device that was current when it
 * was created.
 */
typedef struct prism_b200_host_plan prism_b200_host_plan;

int prism_b200_host_gemm_bf16_create(int M, int N, int K, int block_rows, prism_b200_host_plan** plan);
int prism_b200_host_gemm_bf16_run(prism_b200_host_plan* plan, const uint16_t* A_host, const uint16_t* B_host,
                                  uint16_t* C_host, void* stream);
int prism_b200_host_sgemm_create(int kernel_id, int M, int N, int K, int block_rows, prism_b200_host_plan** plan);
int prism_b200_host_sgemm_run(prism_b200_host_plan* plan, float alpha, const float* A_host, const float* B_host,
                              float beta, float* C_host, void* stream);
int prism_b200_host_scan_create(size_t n, size_t block_elems, prism_b200_host_plan** plan);
int prism_b200_host_scan_run(prism_b200_host_plan* plan, uint32_t* x_host, void* stream);
/* Number of blocks a run is cut into (-1 for a bad handle). */
int prism_b200_host_plan_blocks(const prism_b200_host_plan* plan);
/* Waits for the plan's streams, then frees its buffers, streams and events. */
void prism_b200_host_plan_destroy(prism_b200_host_plan* plan);

#ifdef __cplusplus
}
#endif
#endif /* PRISM_B200_H */
