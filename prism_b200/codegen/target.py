"""`B200CodeGenerator`: the reference's code generator with the sm_100a emissions.

Import only after `prism_b200.codegen.import_prism()` has made the Prism compiler importable.

Overridden or added, each next to the reference emission it stands in for:
  visit_Expr             dispatches `intrinsic.tcgen05_mma`, `intrinsic.tcgen05_commit`, `intrinsic.tmem_ld32`
                         before the reference's `intrinsic.mma` / `intrinsic.wgmma256` (prism/codegen.py:609-625);
  _emit_tcgen05_mma      the counterpart of `_emit_wgmma256` (prism/codegen.py:663-679): where that emits a call of
                         the harness's `wgmma<256, ...>` template, this emits the PTX itself, as `_emit_mma` does for
                         mma.sync (prism/codegen.py:627-661), because one instruction is the whole operation;
  visit_BarrierSetup     the counterpart of prism/codegen.py:904-940 for a tcgen05 pipeline (see the method);
  _emit                  raises the alignment of a kernel's dynamic shared memory from the reference's 128 bytes
                         (prism/codegen.py:365) to 1024: a stage that TMA fills in the 128-byte-swizzled layout and a
                         tcgen05 operand descriptor both need 1024-byte-aligned shared memory.
The waits, expects, arrives and phase flips of the reference (prism/codegen.py:861-902) are emitted unchanged:
they call `wait`, `expect_bytes`, `arrive`, which b200_helpers.py provides under the same names and argument
lists (its `wait` is bounded).
"""
from __future__ import annotations

import ast

from prism.codegen import CodeGenerator

TMEM_COLUMNS = 512   # all of a CTA's tensor memory: two 256-column accumulators

# What a file of generated sm_100a code starts with: the types the emitted signatures name and the flag that
# b200_helpers.wait raises when it gives up.
PRELUDE = """#include <cstdint>
#include <cuda_bf16.h>
#include <cuda.h>

__device__ unsigned int prism_b200_wait_gave_up;   // raised by wait() after about a second without progress
"""


class B200CodeGenerator(CodeGenerator):
    def _emit(self, line: str = "") -> None:
        if line == "extern __shared__ __align__(128) char __smem[];":
            line = "extern __shared__ __align__(1024) char __smem[];"
        super()._emit(line)

    # -- intrinsics ---------------------------------------------------------------------------

    def visit_Expr(self, node: ast.Expr) -> None:
        call = node.value
        if (isinstance(call, ast.Call) and isinstance(call.func, ast.Attribute)
                and isinstance(call.func.value, ast.Name) and call.func.value.id == "intrinsic"):
            handler = {"tcgen05_mma": self._emit_tcgen05_mma, "tcgen05_commit": self._emit_tcgen05_commit,
                       "tmem_ld32": self._emit_tmem_ld32}.get(call.func.attr)
            if handler is not None:
                handler(call)
                return
        super().visit_Expr(node)

    @staticmethod
    def _keyword(node: ast.Call, name: str, default):
        for kw in node.keywords:
            if kw.arg == name:
                return kw.value
        return default

    def _cta_group(self, node: ast.Call) -> int:
        g = self._keyword(node, "cta_group", None)
        value = g.value if isinstance(g, ast.Constant) else 1
        if value not in (1, 2):
            raise ValueError("cta_group must be 1 or 2")
        return value

    def _emit_tcgen05_mma(self, node: ast.Call) -> None:
        """intrinsic.tcgen05_mma(tmem_d, desc_a, desc_b, idesc, accumulate, cta_group=1, kind="f16")

        D[tmem_d] (+)= A[desc_a] * B[desc_b]: tmem_d a 32-bit tensor-memory address, desc_a / desc_b 64-bit
        shared-memory matrix descriptors, idesc the 32-bit instruction descriptor, accumulate 0 to overwrite D.
        Must be reached by exactly one thread of the CTA (of the leader CTA with cta_group=2)."""
        if len(node.args) != 5:
            raise ValueError("intrinsic.tcgen05_mma takes (tmem_d, desc_a, desc_b, idesc, accumulate)")
        tmem_d, desc_a, desc_b, idesc, accumulate = (self._expr(a) for a in node.args)
        kind = self._keyword(node, "kind", None)
        kind = kind.value if isinstance(kind, ast.Constant) else "f16"
        if kind not in ("f16", "tf32", "f8f6f4", "i8"):
            raise ValueError(f"unknown tcgen05.mma kind {kind!r}")
        self._emit("asm volatile(")
        self._indent += 1
        self._emit('"{\\n"')
        self._emit('".reg .pred p;\\n"')
        self._emit('"setp.ne.b32 p, %4, 0;\\n"')
        self._emit(f'"tcgen05.mma.cta_group::{self._cta_group(node)}.kind::{kind} [%0], %1, %2, %3, p;\\n"')
        self._emit('"}\\n"')
        self._emit(f': : "r"({tmem_d}), "l"({desc_a}), "l"({desc_b}), "r"({idesc}), "r"({accumulate})')
        self._emit(': "memory"')
        self._indent -= 1
        self._emit(");")

    def _emit_tcgen05_commit(self, node: ast.Call) -> None:
        """intrinsic.tcgen05_commit(bar, cta_group=1): `bar` (an mbarrier in shared memory) receives one arrival
        once every tcgen05.mma issued so far by this thread has completed.  This is how a stage goes back to the
        producer and how an accumulator is handed to the epilogue."""
        if len(node.args) != 1:
            raise ValueError("intrinsic.tcgen05_commit takes (bar)")
        bar = self._expr(node.args[0])
        self._emit(f'asm volatile("tcgen05.commit.cta_group::{self._cta_group(node)}.mbarrier::arrive::one.shared::cluster.b64 [%0];"')
        self._indent += 1
        self._emit(f': : "r"(static_cast<uint32_t>(__cvta_generic_to_shared({bar}))) : "memory");')
        self._indent -= 1

    def _emit_tmem_ld32(self, node: ast.Call) -> None:
        """intrinsic.tmem_ld32(taddr, out=[r]): 32 consecutive fp32 columns of the calling thread's tensor-memory
        lane into the 32-element uint32_t array r; waits for the load.  Warp-wide (all 32 lanes)."""
        if len(node.args) != 1:
            raise ValueError("intrinsic.tmem_ld32 takes (taddr, out=[r])")
        out = self._keyword(node, "out", None)
        if not isinstance(out, ast.List) or len(out.elts) != 1:
            raise ValueError("intrinsic.tmem_ld32 needs out=[array of 32 uint32_t]")
        r = self._expr(out.elts[0])
        taddr = self._expr(node.args[0])
        regs = ", ".join(f"%{i}" for i in range(32))
        self._emit("asm volatile(")
        self._indent += 1
        self._emit(f'"tcgen05.ld.sync.aligned.32x32b.x32.b32 {{{regs}}}, [%32];\\n"')
        self._emit('"tcgen05.wait::ld.sync.aligned;\\n"')
        self._emit(": " + ", ".join(f'"=r"({r}[{i}])' for i in range(32)))
        self._emit(f': "r"({taddr})')
        self._emit(': "memory"')
        self._indent -= 1
        self._emit(");")

    # -- barriers and tensor memory ---------------------------------------------------------------

    def visit_BarrierSetup(self, node) -> None:
        """Declarations and set-up of a tcgen05 producer/consumer pipeline.

        Against the Hopper emission (prism/codegen.py:904-940):
          * full_i   count 1, as there: the producer's expect_bytes arrival; the TMA bytes complete the phase.
          * empty_i  count 1, not num_consumers: the MMA-issuing thread hands the stage back with ONE
                     tcgen05.commit after its MMAs, whatever the number of epilogue warps.  No initial consumer
                     arrive either: the producer's first wait on a fresh barrier names the parity of the phase
                     "before the first", which is complete by definition (its phase variable starts at 1).
          * acc_full / acc_empty  the accumulator hand-over between the MMA thread (tcgen05.commit) and the
                     num_consumers epilogue warps (one arrive per warp), two accumulators.
          * tensor memory: one warp allocates all 512 columns and writes the base address to shared memory; a
                     tcgen05 fence pair brackets the __syncthreads() that publishes it.  The matching
                     `tmem_dealloc(tmem_base, 512)` is the kernel's last statement (b200_helpers.py).
        """
        n = node.num_slots
        for slot in range(n):
            self._emit(f"__shared__ __align__(8) uint64_t full_{slot}[1];")
        for slot in range(n):
            self._emit(f"__shared__ __align__(8) uint64_t empty_{slot}[1];")
        self._emit("__shared__ __align__(8) uint64_t acc_full[2];")
        self._emit("__shared__ __align__(8) uint64_t acc_empty[2];")
        self._emit("__shared__ uint32_t tmem_slot[1];")
        # phase variables: consumers start at phase 0, the producer's view of "empty" at phase 1
        for slot in range(n):
            self._emit(f"int p{slot} = 0;")
        for slot in range(n):
            self._emit(f"int pe{slot} = 1;")
        self._emit("if (threadIdx.x == 0) {")
        self._indent += 1
        for slot in range(n):
            self._emit(f"init_barrier({self._ctx.block_id}, {self._ctx.thread_id}, __smem, full_{slot}, 0, 1);")
        for slot in range(n):
            self._emit(f"init_barrier({self._ctx.block_id}, {self._ctx.thread_id}, __smem, empty_{slot}, 0, 1);")
        for acc in range(2):
            self._emit(f"init_barrier({self._ctx.block_id}, {self._ctx.thread_id}, __smem, acc_full + {acc}, 0, 1);")
            self._emit(f"init_barrier({self._ctx.block_id}, {self._ctx.thread_id}, __smem, acc_empty + {acc}, 0, {node.num_consumers});")
        self._emit('asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");')
        self._indent -= 1
        self._emit("}")
        self._emit(f"if (({self._ctx.thread_id} / 32) == 1) {{")
        self._indent += 1
        self._emit(f"tmem_alloc({self._ctx.block_id}, {self._ctx.thread_id}, __smem, tmem_slot, {TMEM_COLUMNS});")
        self._indent -= 1
        self._emit("}")
        self._emit(f"tcgen05_fence_before({self._ctx.block_id}, {self._ctx.thread_id}, __smem);")
        self._emit("__syncthreads();")
        self._emit(f"tcgen05_fence_after({self._ctx.block_id}, {self._ctx.thread_id}, __smem);")
        self._emit("const uint32_t tmem_base = tmem_slot[0];")


def generate_b200(func_name: str, auto_sync: bool = False) -> str:
    """`prism.generate` (prism/codegen.py:1000-1025) with `B200CodeGenerator` as the emitter."""
    from prism.registry import registry
    from prism.type_checker import check_function

    found = registry.get(func_name)
    if found is None:
        raise ValueError(f"Function '{func_name}' not found in registry")
    func_type, tree, _ = found
    signature = check_function(func_type, tree)
    if auto_sync:
        from prism.sync_analysis import analyze_sync
        from prism.sync_transform import transform_sync
        plan = analyze_sync(func_type, tree, signature)
        if plan.analyzed:
            tree = transform_sync(tree, plan)
    gen = B200CodeGenerator(func_type, signature)
    gen.visit(tree)
    return gen.get_code()
