"""A whole bf16 GEMM kernel for sm_100a written in the Prism language.

What examples/h100_matmul.py is to the reference's Hopper target, this is to the tcgen05 target: one CTA of 192
threads per 128 x 128 output tile, split by `match split(thread)` into four epilogue warps, a producer warp and an
issuer warp.  The producer's first lane brings 64-wide k-blocks of both operands into two shared-memory stages with
TMA (`load_async` onto the stage's "full" barrier); the issuer's first lane waits for a stage, issues its four
`tcgen05.mma` through `tcgen05_k_block` (whose `tcgen05.commit` frees the stage) and finally signals the accumulator
barrier; the epilogue warps wait for that signal and copy their 32 lanes of tensor memory to D.  Barriers, phases and
tensor memory are declared and handled in the program itself (this target infers none of them).

D[n * M + m] = sum_k B[n, k] * A[m, k] in fp32, stored as bit patterns.  `tiles_n` = N / 128; block b works on tile
(b % tiles_n, b / tiles_n).  The descriptor encodings (`operand_desc`, `IDESC`) are plain CUDA in the file that
make_tile_gemm.py assembles around the emitted text.

Import only after `prism_b200.codegen.import_prism()`; emit with `generate_b200("prism_tile_gemm")`.
"""
from prism import (
    prism, grid, block, thread,
    requires, group, split, partition, claim,
    ptr, const, constexpr, shared, unsafe, attr,
    bf16, uint32_t, uint64_t, CUtensorMap, void,
)


@attr("__launch_bounds__(192, 1)")
@requires(grid[1], block[1], thread[192], smem=122880)
@prism("global")
def prism_tile_gemm(M: int @ grid[1],
                    K: int @ grid[1],
                    tiles_n: int @ grid[1],
                    D: ptr(uint32_t) @ grid[1],
                    tensorMapA: const(CUtensorMap) @ grid[1],
                    tensorMapB: const(CUtensorMap) @ grid[1]):
    with group(grid[1]):
        tile: int @ block[1] = id()
        n0: int @ block[1] = (tile % tiles_n) * 128
        m0: int @ block[1] = (tile / tiles_n) * 128
        num_k: int @ block[1] = K / 64
        # kind::f16 instruction descriptor: D fp32 (bit 4), A and B bf16 (bits 7, 10), both K-major, N >> 3 at bit 17,
        # M >> 4 at bit 24, for a 128 x 128 MMA
        IDESC: constexpr(uint32_t) @ grid[1] = (1 << 4) | (1 << 7) | (1 << 10) | ((128 >> 3) << 17) | ((128 >> 4) << 24)

        with partition(D, p=block[1], offset=n0 * M + m0) as block_D:
            with group(block[1]):
                # two stages of (B block, A block), 16 KB each, in the 128-byte-swizzled K-major layout TMA writes
                stage_b0: shared(bf16[64 * 128], align=1024) @ block[1]
                stage_a0: shared(bf16[64 * 128], align=1024) @ block[1]
                stage_b1: shared(bf16[64 * 128], align=1024) @ block[1]
                stage_a1: shared(bf16[64 * 128], align=1024) @ block[1]
                full_0: shared(uint64_t[1], align=8, static=True) @ block[1]
                full_1: shared(uint64_t[1], align=8, static=True) @ block[1]
                empty_0: shared(uint64_t[1], align=8, static=True) @ block[1]
                empty_1: shared(uint64_t[1], align=8, static=True) @ block[1]
                acc_full: shared(uint64_t[1], align=8, static=True) @ block[1]
                tmem_slot: shared(uint32_t[1], align=8, static=True) @ block[1]

                who: int @ thread[1] = id()
                warp_idx: int @ thread[32] = id()

                # set-up: one thread initialises the barriers, warp 1 allocates tensor memory
                with partition(full_0, p=thread[1], offset=0) as full_0_t:
                    with partition(full_1, p=thread[1], offset=0) as full_1_t:
                        with partition(empty_0, p=thread[1], offset=0) as empty_0_t:
                            with partition(empty_1, p=thread[1], offset=0) as empty_1_t:
                                with partition(acc_full, p=thread[1], offset=0) as acc_full_t:
                                    with group(thread[1]):
                                        if (who == 0):
                                            init_barrier(full_0_t, 0, 1)
                                            init_barrier(full_1_t, 0, 1)
                                            init_barrier(empty_0_t, 0, 1)
                                            init_barrier(empty_1_t, 0, 1)
                                            init_barrier(acc_full_t, 0, 1)
                                            unsafe('asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");')
                with group(thread[32]):
                    if (warp_idx == 1):
                        tmem_alloc(tmem_slot, 512)
                with group(thread[1]):
                    tcgen05_fence_before()
                unsafe("__syncthreads();")
                with group(thread[1]):
                    tcgen05_fence_after()
                tmem_base: uint32_t @ block[1] = tmem_slot[0]

                with claim(block_D, p=thread[128], offset=0) as epi_D:
                    with claim(stage_b0, p=thread[1], offset=0) as b_dst0:
                        with claim(stage_a0, p=thread[1], offset=0) as a_dst0:
                            with claim(stage_b1, p=thread[1], offset=0) as b_dst1:
                                with claim(stage_a1, p=thread[1], offset=0) as a_dst1:
                                    match split(thread):
                                        case 128:
                                            # ---- epilogue: warp w reads lanes 32 (w % 4) .. + 31 of tensor memory ----
                                            quarter: int @ thread[32] = warp_idx % 4
                                            with partition(epi_D, p=thread[32], offset=quarter * 32 * M) as warp_D:
                                                with group(thread[32]):
                                                    lane_e: int @ thread[1] = id()
                                                    with group(thread[1]):
                                                        if (lane_e == 0):
                                                            wait(acc_full, 0)
                                                    unsafe("__syncwarp();")
                                                    with group(thread[1]):
                                                        tcgen05_fence_after()
                                                    for c0 in range(0, 128, 32):
                                                        taddr: uint32_t @ thread[32] = tmem_base + ((quarter * 32) << 16) + c0
                                                        with partition(warp_D, p=thread[32], offset=c0) as out_D:
                                                            tmem_row_to_global(taddr, out_D, M)
                                        case 32:
                                            # ---- producer ----
                                            with group(thread[32]):
                                                lane_p: int @ thread[1] = id()
                                                with group(thread[1]):
                                                    if (lane_p == 0):
                                                        pe0: int @ thread[1] = 1
                                                        pe1: int @ thread[1] = 1
                                                        map_a: ptr(const(void)) @ thread[1]
                                                        map_b: ptr(const(void)) @ thread[1]
                                                        unsafe("map_a = &tensorMapA;")
                                                        unsafe("map_b = &tensorMapB;")
                                                        for kb in range(0, num_k, 2):
                                                            wait(empty_0, pe0)
                                                            pe0 = pe0 ^ 1
                                                            expect_bytes(full_0, 32768)
                                                            load_async(b_dst0, map_b, full_0, kb * 64, n0)
                                                            load_async(a_dst0, map_a, full_0, kb * 64, m0)
                                                            if (kb + 1 < num_k):
                                                                wait(empty_1, pe1)
                                                                pe1 = pe1 ^ 1
                                                                expect_bytes(full_1, 32768)
                                                                load_async(b_dst1, map_b, full_1, (kb + 1) * 64, n0)
                                                                load_async(a_dst1, map_a, full_1, (kb + 1) * 64, m0)
                                        case 32:
                                            # ---- issuer ----
                                            with group(thread[32]):
                                                lane_i: int @ thread[1] = id()
                                                with group(thread[1]):
                                                    if (lane_i == 0):
                                                        p0: int @ thread[1] = 0
                                                        p1: int @ thread[1] = 0
                                                        desc_b0: uint64_t @ thread[1]
                                                        desc_a0: uint64_t @ thread[1]
                                                        desc_b1: uint64_t @ thread[1]
                                                        desc_a1: uint64_t @ thread[1]
                                                        unsafe("desc_b0 = operand_desc(stage_b0); desc_a0 = operand_desc(stage_a0);")
                                                        unsafe("desc_b1 = operand_desc(stage_b1); desc_a1 = operand_desc(stage_a1);")
                                                        for kb in range(0, num_k, 2):
                                                            wait(full_0, p0)
                                                            p0 = p0 ^ 1
                                                            tcgen05_fence_after()
                                                            first: int @ thread[1] = 1
                                                            if (kb == 0):
                                                                first = 0
                                                            tcgen05_k_block(tmem_base, desc_b0, desc_a0, IDESC, first, empty_0)
                                                            if (kb + 1 < num_k):
                                                                wait(full_1, p1)
                                                                p1 = p1 ^ 1
                                                                tcgen05_fence_after()
                                                                tcgen05_k_block(tmem_base, desc_b1, desc_a1, IDESC, 1, empty_1)
                                                        tcgen05_signal(acc_full)

                # ---- tear-down ----
                unsafe("if (prism_b200_wait_gave_up && threadIdx.x == 0) prism_b200_let_loads_land();")
                with group(thread[1]):
                    tcgen05_fence_before()
                unsafe("__syncthreads();")
                with group(thread[32]):
                    if (warp_idx == 1):
                        tmem_dealloc(tmem_base, 512)
    return
