"""The sm_100a code-generation target for the Prism language (prism_b200/codegen): emitted text, as the
reference tests its own generator (test/test_codegen.py never runs a kernel either), plus a cross-compilation of
everything emitted for sm_100a, which is what shows that the tcgen05 / mbarrier / TMA PTX assembles.

Needs a checkout of the Prism compiler (PRISM_REFERENCE, or a sibling directory `reference`); skipped without it.
"""
import ast
import os
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


@pytest.fixture(scope="module")
def cg():
    from prism_b200 import codegen
    try:
        codegen.import_prism()
    except ImportError as e:
        pytest.skip(str(e))
    import warnings
    warnings.simplefilter("ignore")
    from prism_b200.codegen import b200_helpers, b200_mma_step, target  # noqa: F401  (registers the functions)
    return codegen, b200_helpers, target


def test_helpers_keep_the_call_signatures_the_barrier_emission_uses(cg):
    codegen, helpers, target = cg
    text = {name: codegen.generate_b200(name) for name in helpers.HELPERS}
    lead = "int __block_id, int __thread_id, char* __smem"
    assert f"void init_barrier({lead}, uint64_t* bar, int thread_count, int transaction_count)" in text["init_barrier"]
    assert f"void expect_bytes({lead}, uint64_t* bar, int bytes)" in text["expect_bytes"]
    assert f"void arrive({lead}, uint64_t* bar, int count)" in text["arrive"]
    assert f"void wait({lead}, uint64_t* bar, int kPhaseBit)" in text["wait"]
    assert "mbarrier.try_wait.parity" in text["wait"] and "prism_b200_wait_gave_up = 1u" in text["wait"]   # bounded
    assert "bra.uni" not in text["wait"]                                                   # no unbounded spin loop
    assert "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes" in text["load_async"]
    assert "multicast" not in "".join(text.values())
    assert "tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32" in text["tmem_alloc"]
    assert "tcgen05.relinquish_alloc_permit" in text["tmem_alloc"]
    assert "tcgen05.dealloc.cta_group::1.sync.aligned.b32" in text["tmem_dealloc"]


def test_tcgen05_intrinsics_are_emitted_as_ptx(cg):
    codegen, _, _ = cg
    step = codegen.generate_b200("tcgen05_k_block")
    assert "for (int k = 0; k < 4; k++)" in step
    assert "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;" in step
    assert '"r"(tmem_d), "l"((desc_a + (2 * k))), "l"((desc_b + (2 * k))), "r"(idesc), "r"(accumulate)' in step
    assert "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" in step
    assert step.index("tcgen05.mma") < step.index("tcgen05.commit")
    assert "wgmma" not in step
    row = codegen.generate_b200("tmem_row_to_global")
    assert "tcgen05.ld.sync.aligned.32x32b.x32.b32" in row and "tcgen05.wait::ld.sync.aligned" in row
    assert '"=r"(r[0])' in row and '"=r"(r[31])' in row and '"r"(taddr)' in row
    assert "out[lane * stride + c] = r[c];" in row
    sig = codegen.generate_b200("tcgen05_signal")
    assert sig.count("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64") == 1 and "tcgen05.mma" not in sig


def _barrier_setup_text(target, slots, consumers):
    from prism.sync_nodes import BarrierSetup
    gen = target.B200CodeGenerator.__new__(target.B200CodeGenerator)
    from prism.codegen import CodeGenerator
    CodeGenerator.__init__(gen, "global", None)
    gen.visit_BarrierSetup(BarrierSetup(slots, consumers, "thread[128]", "thread[128]", "thread[32]"))
    return gen.get_code()


def test_barrier_setup_for_a_tcgen05_pipeline(cg):
    _, _, target = cg
    text = _barrier_setup_text(target, slots=4, consumers=4)
    for i in range(4):
        assert f"__shared__ __align__(8) uint64_t full_{i}[1];" in text
        assert f"init_barrier(__block_id_0, __thread_id_0, __smem, full_{i}, 0, 1);" in text
        # one tcgen05.commit frees a stage, however many epilogue warps there are
        assert f"init_barrier(__block_id_0, __thread_id_0, __smem, empty_{i}, 0, 1);" in text
        assert f"int p{i} = 0;" in text and f"int pe{i} = 1;" in text
    assert "init_barrier(__block_id_0, __thread_id_0, __smem, acc_empty + 1, 0, 4);" in text   # the epilogue warps
    assert "arrive(" not in text                      # no initial consumer arrive (prism/codegen.py:922-936 has one)
    assert "tmem_alloc(__block_id_0, __thread_id_0, __smem, tmem_slot, 512);" in text
    order = [text.index(s) for s in ("fence.mbarrier_init", "tmem_alloc(", "tcgen05_fence_before(", "__syncthreads();",
                                     "tcgen05_fence_after(", "const uint32_t tmem_base = tmem_slot[0];")]
    assert order == sorted(order)


def test_unknown_kind_and_bad_group_are_refused(cg):
    codegen, _, target = cg
    from prism.codegen import CodeGenerator
    gen = target.B200CodeGenerator.__new__(target.B200CodeGenerator)
    CodeGenerator.__init__(gen, "device", None)
    call = ast.parse("intrinsic.tcgen05_mma(d, a, b, i, acc, kind='fp4')").body[0]
    with pytest.raises(ValueError):
        gen.visit_Expr(call)
    call = ast.parse("intrinsic.tcgen05_commit(bar, cta_group=3)").body[0]
    with pytest.raises(ValueError):
        gen.visit_Expr(call)


def test_everything_emitted_assembles_for_sm_100a(cg, tmp_path):
    """Helpers, the two example functions and a kernel body made of the BarrierSetup emission, one k-block and one
    epilogue read, compiled (not run) with nvcc for sm_100a."""
    codegen, helpers, target = cg
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not found")
    parts = [target.PRELUDE]
    parts += [codegen.generate_b200(name) for name in helpers.HELPERS]
    parts += [codegen.generate_b200("tcgen05_k_block"), codegen.generate_b200("tmem_row_to_global")]
    setup = _barrier_setup_text(target, slots=2, consumers=4)
    parts.append("""
__global__ void __launch_bounds__(192, 1) generated_probe(uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t* out) {
    extern __shared__ char __smem[];
    int __block_id_0 = blockIdx.x;
    int __thread_id_0 = threadIdx.x;
""" + "".join("    " + ln + "\n" for ln in setup.splitlines()) + """
    if (threadIdx.x == 32) {
        tcgen05_k_block(__block_id_0, __thread_id_0, __smem, tmem_base, desc_a, desc_b, idesc, 0, empty_0);
        wait(__block_id_0, __thread_id_0, __smem, empty_0, p0);
    }
    __syncthreads();
    if (threadIdx.x >= 64) {
        const int quarter = (threadIdx.x / 32) & 3;
        tmem_row_to_global(__block_id_0, __thread_id_0, __smem, tmem_base + ((uint32_t)(quarter * 32) << 16), out + quarter * 1024, 32);
    }
    tcgen05_fence_before(__block_id_0, __thread_id_0, __smem);
    __syncthreads();
    if ((threadIdx.x / 32) == 1) tmem_dealloc(__block_id_0, __thread_id_0, __smem, tmem_base, 512);
    (void)pe0; (void)pe1; (void)p1;
}
""")
    src = tmp_path / "generated_b200.cu"
    src.write_text("\n".join(parts))
    r = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-c", str(src), "-o",
                        str(tmp_path / "generated_b200.o")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]


def test_committed_generated_kernel_is_what_the_generator_writes(cg):
    """prism_b200/codegen/generated/tile_gemm.cu is kept in the tree like the reference keeps generated/*.cu; it must
    be exactly what make_tile_gemm.py renders from the Prism programs and the target as they are now."""
    from prism_b200.codegen import make_tile_gemm
    assert make_tile_gemm.OUT.read_text() == make_tile_gemm.render()


def test_generated_kernel_file_names_its_parts():
    """Without the Prism compiler: the committed file has the emitted functions before the hand-written glue, no
    multicast load, no unbounded wait, and compiles for sm_100a."""
    src = ROOT / "prism_b200" / "codegen" / "generated" / "tile_gemm.cu"
    text = src.read_text()
    glue = text.index("// ---------------------------------------------------------------- glue written by hand")
    for name in ("init_barrier", "expect_bytes", "wait", "load_async", "tmem_alloc", "tmem_dealloc", "tcgen05_k_block",
                 "tcgen05_signal", "tmem_row_to_global"):
        assert text.index(f"void {name}(int __block_id, int __thread_id, char* __smem") < glue, name
    assert "tcgen05.mma.cta_group::1.kind::f16" in text[:glue] and "tcgen05.mma" not in text[glue:]
    # the kernel itself is emitted text too, between the two hand-written sections
    kernel = text.index("__global__ __launch_bounds__(192, 1) void prism_tile_gemm(")
    assert glue < kernel < text.index("glue written by hand (host side)")
    body = text[kernel:text.index("glue written by hand (host side)")]
    assert "extern __shared__ __align__(1024) char __smem[];" in body
    for call in ("init_barrier(", "tmem_alloc(", "wait(", "expect_bytes(", "load_async(", "tcgen05_k_block(", "tcgen05_signal(",
                 "tmem_row_to_global(", "tmem_dealloc("):
        assert call in body, call
    assert body.count("if (__thread_id_3 >= 0 && __thread_id_3 < ") == 3          # epilogue, producer and issuer roles
    assert "multicast" not in text and "wgmma" not in text and "prism_b200_wait_gave_up = 1u" in text
    from prism_b200 import build
    assert build.build_generated_tile_gemm(force=True).exists()


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 384, 512), (1024, 512, 2048), (128, 256, 8192), (256, 128, 192)])
def test_generated_kernel_runs_on_the_gpu_and_matches_fp64(shape):
    """The kernel that the generator emitted from the Prism program b200_tile_gemm.py (TMA loads onto mbarriers,
    tcgen05.mma into tensor memory, a commit per stage, tcgen05.ld in the epilogue) on a B200: fp32 sums of exact bf16 products, so every element is within
    K * 2^-23 * sum |b||a| of the fp64 product; on small integers it is exact, which pins the D[n * M + m] layout, the
    operand roles and the order of the stages."""
    import ctypes
    import numpy as np
    import torch
    from oracle import cpu_oracle as O
    from prism_b200 import build
    lib = ctypes.CDLL(str(build.build_generated_tile_gemm()))
    lib.prism_generated_tile_gemm_run.argtypes = [ctypes.c_int] * 3 + [ctypes.c_void_p] * 4
    M, N, K = shape
    dev = "cuda:0"

    def run(A_bits, B_bits):
        a = torch.from_numpy(A_bits.view(np.int16)).to(dev)
        b = torch.from_numpy(B_bits.view(np.int16)).to(dev)
        d = torch.full((N, M), float("nan"), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            assert lib.prism_generated_tile_gemm_run(M, N, K, a.data_ptr(), b.data_ptr(), d.data_ptr(), stream) == 0
            torch.cuda.synchronize()
        assert lib.prism_generated_tile_gemm_gave_up() == 0
        return d.cpu().numpy()

    A, B = O.gemm_bf16_inputs(M, N, K, seed=M + N + K)
    a64, b64 = O.bf16_bits_to_f32(A).astype(np.float64), O.bf16_bits_to_f32(B).astype(np.float64)
    got = run(A, B)
    bound = K * 2.0 ** -23 * (np.abs(b64) @ np.abs(a64).T)
    assert np.all(np.abs(got - b64 @ a64.T) <= bound + 1e-30)
    rng = np.random.default_rng(K)
    Ai = O.f32_to_bf16_bits(rng.integers(-3, 4, (M, K)).astype(np.float32))
    Bi = O.f32_to_bf16_bits(rng.integers(-3, 4, (N, K)).astype(np.float32))
    exact = O.bf16_bits_to_f32(Bi).astype(np.float64) @ O.bf16_bits_to_f32(Ai).astype(np.float64).T
    assert np.array_equal(run(Ai, Bi).astype(np.float64), exact)
    assert lib.prism_generated_tile_gemm_run(100, 128, 64, None, None, None, None) == 1
