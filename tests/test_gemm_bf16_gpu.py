"""GPU parity of the bf16 GEMM through the C ABI: against fp64 NumPy on the
bf16-rounded inputs, |D - D_ref| <= 1e-2 |D_ref| + 1e-2 rms(D_ref), in the
reference's column-major C layout."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from oracle import cpu_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _dev(bits):
    return torch.from_numpy(bits.view(np.int16)).to(DEV).view(torch.bfloat16)


def _assert_symmetric(c_nm: torch.Tensor, c_mn: torch.Tensor):
    """C(A, B)^T == C(B, A), bit for bit: every tile accumulates all of K in one pass, in the same order
    whichever operand indexes the rows."""
    assert torch.equal(c_nm, c_mn.t())


def _run(pb, A_bits, B_bits):
    M, K = A_bits.shape
    N = B_bits.shape[0]
    c = torch.full((N, M), float("nan"), dtype=torch.bfloat16, device=DEV)  # every element must be written
    pb.runmyh100(M, N, K, _dev(A_bits), _dev(B_bits), c)
    torch.cuda.synchronize()
    return c.view(torch.int16).cpu().numpy().view(np.uint16)


# Smallest tile, one of each tile width, several k-blocks (ring wrap), several tiles per CTA,
# non-square, and sizes where M only divides the 128-wide tile.
SHAPES = [(128, 128, 64), (256, 128, 64), (128, 128, 512), (256, 256, 1024), (384, 256, 320), (512, 1024, 256),
          (1024, 512, 2048), (2048, 2048, 2048), (128, 4096, 128), (4096, 128, 192)]


@pytest.mark.parametrize("shape", SHAPES)
def test_matches_fp64_oracle(pb, shape):
    M, N, K = shape
    A, B = O.gemm_bf16_inputs(M, N, K, seed=M * 7 + N * 3 + K)
    out = _run(pb, A, B)
    ok, worst = O.gemm_bf16_check(out, O.gemm_bf16_cpu(A, B))
    assert ok, f"worst error / bound = {worst}"


_CHILD = """
import sys, numpy as np, torch
sys.path.insert(0, %r)
import prism_b200 as pb
from oracle import cpu_oracle as O
worst = 0.0
for (M, N, K) in %r:
    A, B = O.gemm_bf16_inputs(M, N, K, seed=M + N + K)
    a = torch.from_numpy(A.view(np.int16)).cuda().view(torch.bfloat16)
    b = torch.from_numpy(B.view(np.int16)).cuda().view(torch.bfloat16)
    c = torch.full((N, M), float('nan'), dtype=torch.bfloat16, device='cuda')
    pb.runmyh100(M, N, K, a, b, c); torch.cuda.synchronize()
    ok, w = O.gemm_bf16_check(c.view(torch.int16).cpu().numpy().view(np.uint16), O.gemm_bf16_cpu(A, B))
    assert ok, (M, N, K, w)
    worst = max(worst, w)
assert pb.last_error()[0] == 0, pb.last_error()
print('ok', worst)
"""


def test_random_shapes_match_fp64_oracle(pb):
    """Twelve seeded random shapes (M, N multiples of 128, K of 64, up to 1536 x 1536 x 1024)."""
    rng = np.random.default_rng(2718)
    for _ in range(12):
        M, N, K = (int(rng.integers(1, 13)) * 128, int(rng.integers(1, 13)) * 128, int(rng.integers(1, 17)) * 64)
        A, B = O.gemm_bf16_inputs(M, N, K, seed=M + 13 * N + 131 * K)
        ok, worst = O.gemm_bf16_check(_run(pb, A, B), O.gemm_bf16_cpu(A, B))
        assert ok, f"{(M, N, K)}: worst error / bound = {worst}"


@pytest.mark.parametrize("mode,shapes", [
    # one-CTA kernels only
    ("0", [(256, 256, 128), (1024, 1024, 512), (2048, 4096, 256)]),
    # two-CTA kernel, 256 x 256 pair tiles: one tile, several k-blocks (ring wrap), more tiles than pairs
    ("1", [(256, 256, 64), (256, 512, 1024), (1024, 2048, 320), (4096, 4096, 256)]),
    # two-CTA kernel, 512 x 256 pair tiles
    ("2", [(256, 512, 64), (512, 512, 1024), (1024, 2048, 320), (4096, 4096, 256), (2048, 8192, 128)]),
    # the same with the tiles of a partly filled last wave cut into their two n blocks: one tile alone, fewer pieces
    # than pairs, one full wave plus a last wave with two pieces per pair (128 tiles on 74 pairs), 64 tiles, a k-block
    # count that is no multiple of either ring's depth, one k-block, and a shape whose tiles fill the pairs exactly
    ("2/2", [(256, 512, 2048), (1024, 2048, 1024), (2048, 8192, 1024), (1024, 1024, 4160), (1024, 8192, 2048),
             (256, 512, 64), (9472, 1024, 128)]),
    ("2/0", [(1024, 2048, 1024), (2048, 8192, 1024)]),
])
def test_every_kernel_form_forced(mode, shapes):
    """The launcher picks a kernel form by problem size; each form is forced here on small and
    multi-wave shapes (the choice is read from the environment once per process, hence the child)."""
    import os
    import subprocess
    env = dict(os.environ, PRISM_B200_GEMM_PAIR=mode[0])
    if len(mode) > 1:
        env["PRISM_B200_GEMM_FILL"] = mode[2]
    r = subprocess.run([sys.executable, "-c", _CHILD % (str(ROOT), shapes)], env=env, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("shape", [(4096, 8192, 8192), (2048, 8192, 8192), (4096, 4096, 4096)])
def test_filling_the_last_wave_changes_no_bit(pb, shape):
    """The benchmark shape cut over 2 and 4 GPUs, and 4096^3 (256, 128 and 128 tiles of 512 x 256 on 74 pairs): with the
    last wave's tiles computed whole or as their two n blocks, and with the launcher's own choice, the output is the
    same bit for bit, since every piece accumulates all of K in the order the whole tile does."""
    M, N, K = shape
    lib = pb.load()
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    a = torch.randn((M, K), device=DEV, generator=g).to(torch.bfloat16)
    b = torch.randn((N, K), device=DEV, generator=g).to(torch.bfloat16)
    outs = {}
    try:
        for mode in (0, 2, -1):
            assert lib.prism_b200_gemm_bf16_fill_mode(mode) == 0
            c = torch.full((N, M), float("nan"), dtype=torch.bfloat16, device=DEV)
            pb.runmyh100(M, N, K, a, b, c)
            torch.cuda.synchronize()
            assert pb.last_error()[0] == 0, pb.last_error()
            outs[mode] = c.view(torch.int16)
    finally:
        lib.prism_b200_gemm_bf16_fill_mode(-1)
    for mode in (2, -1):
        assert torch.equal(outs[0], outs[mode]), f"fill mode {mode} differs from the unfilled kernel"
    rows = [0, 127, 128, 255, 256, 383, 384, 511, N - 1]
    ref = (b[rows].double() @ a.double().t()).cpu().numpy()
    got = outs[0].view(torch.bfloat16)[rows].double().cpu().numpy()
    rms = float(np.sqrt(np.mean(ref * ref)))
    assert np.all(np.abs(got - ref) <= 1e-2 * np.abs(ref) + 1e-2 * rms)


def test_layout_is_column_major_and_exact_on_small_integers(pb):
    """Integer-valued inputs with small K: every product and sum is exact in fp32 and in bf16,
    so the result must equal the oracle bit for bit, which also pins the C[n * M + m] layout."""
    M, N, K = 256, 384, 64
    rng = np.random.default_rng(1)
    A = O.f32_to_bf16_bits(rng.integers(-2, 3, (M, K)).astype(np.float32))
    B = O.f32_to_bf16_bits(rng.integers(-2, 3, (N, K)).astype(np.float32))
    out = _run(pb, A, B)
    ref = O.gemm_bf16_cpu(A, B)
    assert np.array_equal(O.bf16_bits_to_f32(out).reshape(N, M), ref.astype(np.float32))


def test_many_tiles_per_cta_4096(pb):
    """4096^3: 512 tiles over 148 CTAs -> several tiles per CTA, both accumulators and every ring stage reused.
    Checked on sampled rows in fp64 and against the full-size property C(A, B)^T == C(B, A)."""
    S = 4096
    A, B = O.gemm_bf16_inputs(S, S, S, seed=4096)
    out = O.bf16_bits_to_f32(_run(pb, A, B)).reshape(S, S)          # [n, m]
    swapped = O.bf16_bits_to_f32(_run(pb, B, A)).reshape(S, S)      # [m, n]
    _assert_symmetric(torch.from_numpy(out), torch.from_numpy(swapped))
    rows = [0, 1, 127, 128, 129, 2047, 2048, 4095]
    a = O.bf16_bits_to_f32(A).astype(np.float64)
    b = O.bf16_bits_to_f32(B).astype(np.float64)
    ref = b[rows] @ a.T                                               # [n in rows, m]
    rms = float(np.sqrt(np.mean(ref * ref)))
    assert np.all(np.abs(out[rows] - ref) <= 1e-2 * np.abs(ref) + 1e-2 * rms)


def test_row_major_output_is_the_exchanged_call(pb):
    M, N, K = 384, 640, 192
    A, B = O.gemm_bf16_inputs(M, N, K, seed=21)
    a = torch.from_numpy(A.view(np.int16)).view(torch.bfloat16).to(DEV)
    b = torch.from_numpy(B.view(np.int16)).view(torch.bfloat16).to(DEV)
    col = pb.gemm_bf16(a, b)                     # (N, M): the reference's column-major C
    row = pb.gemm_bf16(a, b, row_major=True)     # (M, N)
    torch.cuda.synchronize()
    assert row.shape == (M, N) and torch.equal(row, col.t())
    ref = O.gemm_bf16_cpu(A, B).T
    rms = float(np.sqrt(np.mean(ref * ref)))
    assert np.all(np.abs(row.float().cpu().numpy() - ref) <= 1e-2 * np.abs(ref) + 1e-2 * rms)


def test_benchmark_size_8192(pb):
    """8192^3, the headline configuration (512 x 256 two-CTA tiles, 6.9 waves): sampled rows against fp64
    and the full-size symmetry C(A, B)^T == C(B, A), which the swapped call computes with the roles of the
    lane and column operands exchanged."""
    S = 8192
    g = torch.Generator(device=DEV).manual_seed(8192)
    a = (torch.randn((S, S), device=DEV, generator=g) * 0.1).to(torch.bfloat16)
    b = (torch.randn((S, S), device=DEV, generator=g) * 0.1).to(torch.bfloat16)
    c = torch.full((S, S), float("nan"), dtype=torch.bfloat16, device=DEV)
    c2 = torch.full((S, S), float("nan"), dtype=torch.bfloat16, device=DEV)
    pb.runmyh100(S, S, S, a, b, c)      # c[n, m]
    pb.runmyh100(S, S, S, b, a, c2)     # c2[m, n]
    torch.cuda.synchronize()
    _assert_symmetric(c, c2)
    rows = [0, 1, 127, 128, 255, 256, 511, 512, 4095, 4096, 8191]
    ref = (b[rows].double() @ a.double().t()).cpu().numpy()         # [n in rows, m]
    got = c[rows].double().cpu().numpy()
    rms = float(np.sqrt(np.mean(ref * ref)))
    assert np.all(np.abs(got - ref) <= 1e-2 * np.abs(ref) + 1e-2 * rms)


@pytest.mark.parametrize("shape", [(6144, 6144, 6144), (12288, 12288, 12288), (12288, 6144, 2048), (16384, 16384, 1024)])
def test_sweep_sizes_of_the_reference_harness(pb, shape):
    """Sizes of the reference's sweep (evals/run_h100.sh:12) that are not powers of two, and the largest one:
    tile counts that leave a partly filled last wave.  Sampled rows of both CTA ranks and both row blocks of a
    512-row tile against fp64, plus the full-size symmetry C(A, B)^T == C(B, A)."""
    M, N, K = shape
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    a = (torch.randn((M, K), device=DEV, generator=g) * 0.1).to(torch.bfloat16)
    b = (torch.randn((N, K), device=DEV, generator=g) * 0.1).to(torch.bfloat16)
    c = torch.full((N, M), float("nan"), dtype=torch.bfloat16, device=DEV)
    c2 = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    pb.runmyh100(M, N, K, a, b, c)      # c[n, m]
    pb.runmyh100(N, M, K, b, a, c2)     # c2[m, n]
    torch.cuda.synchronize()
    _assert_symmetric(c, c2)
    rows = [0, 127, 128, 255, 256, 383, 384, 511, 512, N // 2 - 1, N // 2, N - 129, N - 1]
    ref = (b[rows].double() @ a.double().t()).cpu().numpy()         # [n in rows, m]
    got = c[rows].double().cpu().numpy()
    rms = float(np.sqrt(np.mean(ref * ref)))
    assert np.all(np.abs(got - ref) <= 1e-2 * np.abs(ref) + 1e-2 * rms)


@pytest.mark.parametrize("shape,alpha,beta", [((128, 128, 64), 1.0, 0.0), ((256, 384, 192), 1.5, 0.5), ((1024, 512, 2048), -0.75, 2.0),
                                              ((384, 1280, 320), 0.0, 1.0), ((2048, 2048, 1024), 2.0, -1.0)])
def test_alpha_beta_epilogue_matches_fp64_oracle(pb, shape, alpha, beta):
    """D = alpha * A * B^T + beta * C, out of place and in place."""
    M, N, K = shape
    A, B = O.gemm_bf16_inputs(M, N, K, seed=M + 2 * N + 3 * K)
    rng = np.random.default_rng(M * N)
    C = O.f32_to_bf16_bits(rng.standard_normal((N, M)).astype(np.float32))
    ref = O.gemm_bf16_axpby_cpu(alpha, A, B, beta, C)
    a, b, c = _dev(A), _dev(B), _dev(C).reshape(N, M)
    d = torch.full((N, M), float("nan"), dtype=torch.bfloat16, device=DEV)
    pb.gemm_bf16_axpby(alpha, a, b, beta, c, out=d)
    torch.cuda.synchronize()
    ok, worst = O.gemm_bf16_check(d.view(torch.int16).cpu().numpy().view(np.uint16), ref)
    assert ok, f"worst error / bound = {worst}"
    assert torch.equal(c, _dev(C).reshape(N, M)), "the input C was modified by the out-of-place call"
    pb.gemm_bf16_axpby(alpha, a, b, beta, c)          # in place
    torch.cuda.synchronize()
    assert torch.equal(c, d)
    if alpha == 1.0 and beta == 0.0:                  # the plain product, bit for bit
        assert torch.equal(d, pb.gemm_bf16(a, b))


def test_agrees_with_cublas_like_the_reference_harness(pb):
    """The reference harness accepts |kernel - cuBLAS| <= 0.1 (evals/h100_bench/main.cu:43-55); same check here."""
    M, N, K = 1024, 1024, 1024
    A, B = O.gemm_bf16_inputs(M, N, K, seed=2)
    out = O.bf16_bits_to_f32(_run(pb, A, B)).reshape(N, M)
    lib = (_dev(B).float() @ _dev(A).float().t()).cpu().numpy()
    assert np.max(np.abs(out - lib)) <= 0.1


def test_rejects_unsupported_shapes_and_alignment(pb):
    a = torch.zeros(128 * 64 + 8, dtype=torch.bfloat16, device=DEV)
    c = torch.zeros(128 * 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(pb.PrismB200Error) as e:
        pb.runmyh100(100, 128, 64, a, a, c)
    assert e.value.code == 2
    with pytest.raises(pb.PrismB200Error) as e:
        pb.runmyh100(128, 128, 32, a, a, c)
    assert e.value.code == 2
    with pytest.raises(pb.PrismB200Error) as e:
        pb.runmyh100(128, 128, 64, a[1:], a, c)
    assert e.value.code == 3
    pb.clear_error()


def test_new_buffer_same_shape_is_not_served_a_stale_map(pb):
    """The reference caches its tensor maps on M alone (evals/h100_bench/utils.cuh:512-518)."""
    M = N = K = 256
    A1, B1 = O.gemm_bf16_inputs(M, N, K, seed=10)
    A2, B2 = O.gemm_bf16_inputs(M, N, K, seed=11)
    o1 = _run(pb, A1, B1)
    o2 = _run(pb, A2, B2)
    assert O.gemm_bf16_check(o1, O.gemm_bf16_cpu(A1, B1))[0]
    assert O.gemm_bf16_check(o2, O.gemm_bf16_cpu(A2, B2))[0]
