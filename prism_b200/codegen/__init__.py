"""A Blackwell (sm_100a) code-generation target for the Prism language.

The reference emits its Hopper bf16 kernel from a Prism program: `intrinsic.wgmma256(...)` becomes a
`wgmma<256, ...>` call (prism/codegen.py:663-679), and the barrier declarations, initialisation, waits and
arrives are inferred by its sync passes and emitted from `BarrierSetup` and its sibling nodes
(prism/codegen.py:904-940, prism/sync_transform.py:518-730).  `wgmma` does not exist on sm_100a; its place is
taken by `tcgen05.mma` with accumulators in tensor memory, which changes three things a Prism program sees:

  * the MMA is issued by ONE thread and names a tensor-memory address, two shared-memory descriptors and an
    instruction descriptor                  -> `intrinsic.tcgen05_mma(...)`, emitted as inline PTX;
  * a stage is handed back to the producer by `tcgen05.commit` arriving on the stage's "empty" barrier once,
    not by every consumer warp arriving      -> `intrinsic.tcgen05_commit(bar)`, and `BarrierSetup` initialises the
    empty barriers with count 1 and needs no initial consumer arrive;
  * tensor memory has to be allocated by one warp, published through shared memory, and freed before the CTA
    exits                                     -> `BarrierSetup` also emits the allocation and the base address, and
    `intrinsic.tmem_ld32(...)` reads an accumulator row for the epilogue;
  * swizzled TMA stages and tcgen05 operand descriptors need 1024-byte-aligned shared memory
                                              -> a kernel's dynamic shared memory is declared with that alignment.

What is here:
  target.py        `B200CodeGenerator`, a subclass of the reference's `CodeGenerator` with those emissions, and
                   `generate_b200(name, auto_sync=False)`, the counterpart of `prism.generate`.
  b200_helpers.py  the device helpers a generated kernel calls (mbarrier init / expect / arrive / bounded wait,
                   2-D TMA load, tensor-memory alloc / free, tcgen05 fences), written in the Prism language
                   like the reference's examples/h100_helpers.py and emitted by the reference's own generator.
  b200_mma_step.py small Prism programs on the new intrinsics: the four MMAs of one 64-wide k-block with the commit
                   that frees the stage, the commit that tells the epilogue a tile is complete, and the read of an
                   accumulator row out of tensor memory.
  b200_tile_gemm.py  a whole kernel in the Prism language: a bf16 GEMM, one 128 x 128 tile per CTA, whose 192 threads
                   `match split(thread)` divides into epilogue warps, a TMA producer and a tcgen05.mma issuer.
  make_tile_gemm.py  writes generated/tile_gemm.cu: that kernel and everything it calls, as emitted, plus a hand-written
                   host launcher -- kept in the tree like the reference's generated/*.cu; a GPU test compares its
                   output with the product in float64.

The Prism compiler itself is not part of this package: `import_prism()` puts a checkout of it on the path
(argument, else the environment variable PRISM_REFERENCE, else a sibling directory `reference`).  Nothing on
the kernel path of `prism_b200` imports this sub-package; it produces CUDA source text, which
tests/test_codegen_b200.py checks, cross-compiles for sm_100a and, for generated/tile_gemm.cu, runs on the GPU.
"""
from __future__ import annotations

import importlib
import os
import sys
from pathlib import Path


def import_prism(path: str | os.PathLike | None = None):
    """Import the Prism compiler (`prism`) from a checkout of manya-bansal/prism and return the module."""
    if "prism" in sys.modules and hasattr(sys.modules["prism"], "generate"):
        return sys.modules["prism"]
    root = Path(path or os.environ.get("PRISM_REFERENCE") or Path(__file__).resolve().parents[3] / "reference")
    if not (root / "prism" / "codegen.py").exists():
        raise ImportError(f"no Prism checkout at {root}; pass its path or set PRISM_REFERENCE")
    if str(root) not in sys.path:
        sys.path.insert(0, str(root))
    return importlib.import_module("prism")


def generate_b200(func_name: str, auto_sync: bool = False, prism_path=None) -> str:
    """CUDA source of a registered Prism function, emitted by the sm_100a target (see target.py)."""
    import_prism(prism_path)
    from .target import generate_b200 as _generate
    return _generate(func_name, auto_sync)
