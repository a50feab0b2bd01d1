"""A Prism program on the sm_100a target: the MMAs of one 64-wide k-block of a bf16 tile.

What `intrinsic.wgmma256(...)` inside `wgmma_async` is to the reference's Hopper kernel
(examples/h100_matmul.py:20-297), this is to a tcgen05 kernel: one thread issues four
`tcgen05.mma` of K = 16 each over a stage that TMA has written in the 128-byte-swizzled K-major
layout (16 bf16 = 32 bytes further along K is +2 in a descriptor's address field), then hands the
stage back to the producer with one `tcgen05.commit` on its "empty" barrier.  `first` is 0 for a
tile's first k-block, whose first MMA overwrites the accumulator instead of adding to it.

Import only after `prism_b200.codegen.import_prism()`; emit with `generate_b200("tcgen05_k_block")`.
"""
from prism import (
    prism, block, thread,
    requires, group,
    ptr, attr, unsafe, uint32_t, uint64_t, intrinsic,
)


@attr("static __forceinline__")
@requires(thread[1])
@prism("device")
def tcgen05_k_block(tmem_d: uint32_t @ thread[1],
                    desc_a: uint64_t @ thread[1],
                    desc_b: uint64_t @ thread[1],
                    idesc: uint32_t @ thread[1],
                    first: int @ thread[1],
                    empty_bar: ptr(uint64_t) @ block[1]):
    with group(thread[1]):
        for k in range(0, 4, 1):
            accumulate: int @ thread[1] = first + k
            intrinsic.tcgen05_mma(tmem_d, desc_a + 2 * k, desc_b + 2 * k, idesc, accumulate, cta_group=1, kind="f16")
        intrinsic.tcgen05_commit(empty_bar, cta_group=1)
    return


# Tells the epilogue that a tile is complete: one tcgen05.commit on the accumulator's "full" barrier, which arrives
# once every MMA issued so far by this thread has finished.  (A comment, not a docstring: the generator would emit a
# string statement as code.)
@attr("static __forceinline__")
@requires(thread[1])
@prism("device")
def tcgen05_signal(bar: ptr(uint64_t) @ block[1]):
    with group(thread[1]):
        intrinsic.tcgen05_commit(bar, cta_group=1)
    return


# Epilogue step: 32 fp32 columns of each lane's accumulator row, from tensor memory to `out` (lane l writes 32
# consecutive words at out + l * stride), as bit patterns.
@attr("static __forceinline__")
@requires(thread[32])
@prism("device")
def tmem_row_to_global(taddr: uint32_t @ thread[32],
                       out: ptr(uint32_t) @ thread[32],
                       stride: int @ thread[32]):
    with group(thread[32]):
        lane: int @ thread[1] = id()
        r: uint32_t[32] @ thread[1]
        intrinsic.tmem_ld32(taddr, out=[r])
        for c in range(0, 32, 1):
            unsafe("out[lane * stride + c] = r[c];")
    return
