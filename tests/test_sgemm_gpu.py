"""GPU parity of the SGEMM family through the C ABI: against fp64 NumPy (norm-wise
relative error <= 1e-5), against the reference's kernels recompiled for sm_100,
and against the GPU-generated fixture."""
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
KERNELS = [1, 2, 3, 4, 5, 6]


def _run(pb, k, alpha, A, B, beta, C):
    a, b, c = (torch.from_numpy(t).to(DEV) for t in (A, B, C))
    pb.run_my_kernel(k, A.shape[0], B.shape[1], A.shape[1], alpha, a, b, beta, c)
    torch.cuda.synchronize()
    return c.cpu().numpy()


@pytest.mark.parametrize("k", KERNELS)
def test_config1_1024_alpha1_beta0(pb, k):
    """M=N=K=1024, alpha=1, beta=0, C zero-initialised."""
    A, B, C = O.sgemm_inputs(1024, 1024, 1024, seed=1, zero_c=True)
    out = _run(pb, k, 1.0, A, B, 0.0, C)
    assert O.sgemm_rel_error(out, O.sgemm_cpu(1.0, A, B, 0.0, C)) <= O.SGEMM_TOL


@pytest.mark.parametrize("k", KERNELS)
def test_config3_1024_alpha15_beta05(pb, k):
    A, B, C = O.sgemm_inputs(1024, 1024, 1024, seed=3)
    out = _run(pb, k, 1.5, A, B, 0.5, C)
    assert O.sgemm_rel_error(out, O.sgemm_cpu(1.5, A, B, 0.5, C)) <= O.SGEMM_TOL


@pytest.mark.parametrize("k", [4, 5])
def test_config3_2048(pb, k):
    A, B, C = O.sgemm_inputs(2048, 2048, 2048, seed=32)
    out = _run(pb, k, 1.5, A, B, 0.5, C)
    assert O.sgemm_rel_error(out, O.sgemm_cpu(1.5, A, B, 0.5, C)) <= O.SGEMM_TOL


@pytest.mark.parametrize("shape", [(128, 128, 32), (128, 256, 64), (256, 128, 96), (384, 640, 160), (128, 128, 4096)])
def test_kernel5_tile_edges(pb, shape):
    M, N, K = shape
    A, B, C = O.sgemm_inputs(M, N, K, seed=M + N + K)
    out = _run(pb, 5, -0.75, A, B, 2.0, C)
    assert O.sgemm_rel_error(out, O.sgemm_cpu(-0.75, A, B, 2.0, C)) <= O.SGEMM_TOL


def test_kernel5_more_tiles_than_resident_ctas(pb):
    """18 x 18 = 324 tiles on 296 resident CTAs: a second, partly filled wave."""
    M = N = 2304
    K = 96
    A, B, C = O.sgemm_inputs(M, N, K, seed=2304)
    out = _run(pb, 5, 1.5, A, B, 0.5, C)
    assert O.sgemm_rel_error(out, O.sgemm_cpu(1.5, A, B, 0.5, C)) <= O.SGEMM_TOL


def test_kernel5_scalar_and_packed_fma_agree(pb, monkeypatch):
    """fma.rn.f32x2 is two independent fp32 FMAs: both forms of kernel 5 must agree bit for bit.
    (The scalar form is selected by an environment variable read at first use, so it is run in a child.)"""
    import subprocess
    code = (
        "import sys, numpy as np, torch; sys.path.insert(0, %r)\n"
        "import prism_b200 as pb\n"
        "from oracle import cpu_oracle as O\n"
        "A,B,C = O.sgemm_inputs(256, 384, 512, seed=11)\n"
        "a,b,c = (torch.from_numpy(t).cuda() for t in (A,B,C))\n"
        "pb.run_my_kernel(5, 256, 384, 512, 1.5, a, b, 0.5, c); torch.cuda.synchronize()\n"
        "np.save(sys.argv[1], c.cpu().numpy())\n" % str(ROOT))
    outs = []
    for scalar in ("0", "1"):
        path = f"/tmp/prism_b200_k5_{scalar}.npy"
        env = dict(**__import__("os").environ, PRISM_B200_SGEMM_SCALAR=scalar)
        subprocess.run([sys.executable, "-c", code, path], check=True, env=env, timeout=300)
        outs.append(np.load(path))
    assert np.array_equal(outs[0], outs[1])


def test_kernel5_every_tile_form(pb):
    """Kernel 5 has 128 x 128, 64 x 128 and 64 x 64 tiles and picks by an estimate of the makespan, so 1152 x 1152, its
    top 512 rows and its top 256 rows need not run the same form (K = 80 is no multiple of 32, so no tile is shared
    along K here).  All are checked against fp64 and, having the same k order per element, against each other bit for
    bit.  Then each form is forced on the whole matrix."""
    M, N, K = 1152, 1152, 80
    A, B, C = O.sgemm_inputs(M, N, K, seed=1152)
    big = _run(pb, 5, 1.5, A, B, 0.5, C)
    assert O.sgemm_rel_error(big, O.sgemm_cpu(1.5, A, B, 0.5, C)) <= O.SGEMM_TOL
    for rows in (512, 256):
        small = _run(pb, 5, 1.5, A[:rows].copy(), B, 0.5, C[:rows].copy())
        assert np.array_equal(big[:rows], small), rows
    lib = pb.load()
    try:
        for mode in (0, 1, 2):
            assert lib.prism_b200_sgemm_tile_mode(mode) == 0
            assert np.array_equal(_run(pb, 5, 1.5, A, B, 0.5, C), big), mode
        assert lib.prism_b200_sgemm_tile_mode(3) == 1
        pb.clear_error()
    finally:
        lib.prism_b200_sgemm_tile_mode(-1)


@pytest.mark.parametrize("form", [1, 2])
@pytest.mark.parametrize("K", [1024, 1056, 1040])
def test_kernel5_tiles_shared_along_k(pb, form, K):
    """Clusters of 2 or 4 CTAs multiply one range of K each and add their partial tiles through distributed shared
    memory.  K = 1024 divides for 2 and 4 CTAs, 1056 = 16 * 66 only for 2 (a request for 4 runs with 2), 1040 = 16 * 65 for
    neither (runs unshared).  Every result is within the bound of fp64, equal on a second run bit for bit, and -- on
    small integers, where every sum is exact -- equal to the exact product, which pins which CTA writes which rows."""
    M, N = 384, 640                    # multiples of 128: kernel 5's tiled forms (6 x 5 or 6 x 10 tiles)
    A, B, C = O.sgemm_inputs(M, N, K, seed=K + form)
    ref = O.sgemm_cpu(1.5, A, B, 0.5, C)
    rng = np.random.default_rng(K)
    Ai, Bi, Ci = (rng.integers(-2, 3, shp).astype(np.float32) for shp in ((M, K), (K, N), (M, N)))
    exact = (Ai.astype(np.float64) @ Bi.astype(np.float64) + Ci).astype(np.float32)
    lib = pb.load()
    outs = {}
    try:
        assert lib.prism_b200_sgemm_tile_mode(form) == 0
        for slices in (1, 2, 4):
            assert lib.prism_b200_sgemm_k_slices(slices) == 0
            out = _run(pb, 5, 1.5, A, B, 0.5, C)
            assert O.sgemm_rel_error(out, ref) <= O.SGEMM_TOL, slices
            assert np.array_equal(out, _run(pb, 5, 1.5, A, B, 0.5, C)), slices
            assert np.array_equal(_run(pb, 5, 1.0, Ai, Bi, 1.0, Ci), exact), slices
            outs[slices] = out
        assert lib.prism_b200_sgemm_k_slices(3) == 1
        pb.clear_error()
    finally:
        lib.prism_b200_sgemm_tile_mode(-1)
        lib.prism_b200_sgemm_k_slices(-1)
    if K == 1024:
        assert not np.array_equal(outs[1], outs[2])    # the shared forms did run: each range of K is rounded on its own
    if K == 1056:
        assert np.array_equal(outs[2], outs[4])        # four CTAs do not divide K: two are used
    if K == 1040:
        assert np.array_equal(outs[1], outs[2]) and np.array_equal(outs[1], outs[4])


@pytest.mark.parametrize("k", KERNELS)
@pytest.mark.parametrize("shape", [(1, 1, 1), (33, 65, 17), (100, 130, 50), (129, 127, 31), (64, 64, 0)])
def test_ragged_shapes_every_kernel(pb, k, shape):
    """Shapes no tile divides, and K = 0 (C = beta * C)."""
    M, N, K = shape
    A, B, C = O.sgemm_inputs(M, N, max(K, 1), seed=7)
    A, B = A[:, :K].copy(), B[:K].copy()
    out = _run(pb, k, 1.5, A, B, 0.5, C)
    assert O.sgemm_rel_error(out, O.sgemm_cpu(1.5, A, B, 0.5, C)) <= O.SGEMM_TOL


def test_random_ragged_shapes(pb):
    """Twenty seeded random shapes up to 400 x 400 x 300, every kernel id, random alpha and beta."""
    rng = np.random.default_rng(31415)
    for it in range(20):
        M, N, K = (int(v) for v in rng.integers(1, (401, 401, 301)))
        alpha, beta = float(rng.uniform(-2, 2)), float(rng.uniform(-2, 2))
        A, B, C = O.sgemm_inputs(M, N, K, seed=1000 + it)
        ref = O.sgemm_cpu(alpha, A, B, beta, C)
        for k in KERNELS:
            out = _run(pb, k, alpha, A, B, beta, C)
            assert O.sgemm_rel_error(out, ref) <= O.SGEMM_TOL, (k, M, N, K)


def test_kernel5_random_tiled_shapes(pb):
    """Shapes that kernel 5's tiled forms take (M, N multiples of 128, K of 16), both tile forms."""
    rng = np.random.default_rng(1618)
    for it in range(8):
        M, N, K = int(rng.integers(1, 12)) * 128, int(rng.integers(1, 12)) * 128, int(rng.integers(1, 20)) * 16
        A, B, C = O.sgemm_inputs(M, N, K, seed=2000 + it)
        out = _run(pb, 5, 1.5, A, B, 0.5, C)
        assert O.sgemm_rel_error(out, O.sgemm_cpu(1.5, A, B, 0.5, C)) <= O.SGEMM_TOL, (M, N, K)


def test_linearity_at_4096(pb):
    """Benchmark size, checked without an fp64 4096^3 product: rows sampled against fp64, plus
    C(alpha=2, beta=0) == 2 * C(alpha=1, beta=0) exactly (scaling by 2 is exact in fp32)."""
    S = 4096
    A, B, C = O.sgemm_inputs(S, S, S, seed=4096, zero_c=True)
    a, b = torch.from_numpy(A).to(DEV), torch.from_numpy(B).to(DEV)
    c1 = torch.zeros(S, S, device=DEV)
    c2 = torch.zeros(S, S, device=DEV)
    pb.run_my_kernel(5, S, S, S, 1.0, a, b, 0.0, c1)
    pb.run_my_kernel(5, S, S, S, 2.0, a, b, 0.0, c2)
    torch.cuda.synchronize()
    assert torch.equal(c2, 2.0 * c1)
    rows = [0, 1, 127, 128, 2047, 3583, 3584, 3999, 4095]
    ref = A[rows].astype(np.float64) @ B.astype(np.float64)
    got = c1[rows].cpu().numpy()
    assert O.sgemm_rel_error(got, ref) <= O.SGEMM_TOL


def test_sweep_size_8192_sampled(pb):
    """Largest size of the sweep: rows sampled against fp64 (inputs generated on the device)."""
    S = 8192
    g = torch.Generator(device=DEV).manual_seed(81920)
    a = torch.rand((S, S), device=DEV, generator=g) * 2 - 1
    b = torch.rand((S, S), device=DEV, generator=g) * 2 - 1
    c0 = torch.rand((S, S), device=DEV, generator=g) * 2 - 1
    c = c0.clone()
    pb.run_my_kernel(5, S, S, S, 1.5, a, b, 0.5, c)
    torch.cuda.synchronize()
    rows = [0, 127, 128, 4095, 4096, 8064, 8191]
    ref = (1.5 * (a[rows].double() @ b.double()) + 0.5 * c0[rows].double()).cpu().numpy()
    assert O.sgemm_rel_error(c[rows].cpu().numpy(), ref) <= O.SGEMM_TOL


def test_kernel5_misaligned_operand_takes_the_checked_kernel(pb):
    """A pointer that is not 16-byte aligned cannot use the 16-byte-vector kernel; the dispatcher must not reject it."""
    M = N = K = 256
    A, B, C = O.sgemm_inputs(M, N, K, seed=77)
    buf = torch.empty(M * K + 1, dtype=torch.float32, device=DEV)
    a = buf[1:]
    a.copy_(torch.from_numpy(A).reshape(-1))
    b, c = torch.from_numpy(B).to(DEV), torch.from_numpy(C).to(DEV)
    assert a.data_ptr() % 16 != 0
    pb.run_my_kernel(5, M, N, K, 1.5, a, b, 0.5, c)
    torch.cuda.synchronize()
    assert O.sgemm_rel_error(c.cpu().numpy(), O.sgemm_cpu(1.5, A, B, 0.5, C)) <= O.SGEMM_TOL


@pytest.mark.parametrize("k", [1, 2, 3, 4, 5])
def test_matches_reference_kernels(pb, ref_gpu, k):
    """Side by side with the reference's generated kernel k (recompiled for sm_100, harness launch geometry)."""
    M = N = K = 512
    A, B, C = O.sgemm_inputs(M, N, K, seed=50 + k)
    mine = _run(pb, k, 1.5, A, B, 0.5, C)
    a, b, c = (torch.from_numpy(t).to(DEV) for t in (A, B, C))
    torch.cuda.synchronize()
    assert ref_gpu.ref_sgemm(k, M, N, K, 1.5, a.data_ptr(), b.data_ptr(), 0.5, c.data_ptr()) == 0
    torch.cuda.synchronize()
    theirs = c.cpu().numpy()
    ref64 = O.sgemm_cpu(1.5, A, B, 0.5, C)
    assert O.sgemm_rel_error(theirs, ref64) <= O.SGEMM_TOL      # the reference itself meets the bound
    assert O.sgemm_rel_error(mine, ref64) <= O.SGEMM_TOL
    assert O.sgemm_rel_error(mine, theirs.astype(np.float64)) <= 2 * O.SGEMM_TOL


def test_golden_fixture_from_reference_kernels(pb):
    path = ROOT / "tests" / "golden" / "sgemm_ref_gpu.npz"
    if not path.exists():
        pytest.skip("GPU-generated fixture not present")
    g = np.load(path)
    for k in (1, 2, 3, 4, 5):
        out = _run(pb, k, float(g["alpha"]), g["A"], g["B"], float(g["beta"]), g["C"].copy())
        assert O.sgemm_rel_error(out, g[f"out_k{k}"].astype(np.float64)) <= 2 * O.SGEMM_TOL, k
