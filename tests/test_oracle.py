"""The CPU oracle against itself, against the reference's own CPU loop and against the committed fixtures."""
import ctypes
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from oracle import cpu_oracle as O  # noqa: E402

GOLDEN = ROOT / "tests" / "golden"


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


@pytest.mark.parametrize("n", [0, 1, 5, 31, 32, 33, 1000, 4096, 4097, 16384, 50001])
def test_scan_numpy_matches_literal_loop(n):
    x = O.scan_inputs(n, seed=n + 1, high=1 << 31)  # large values: exercises wrap-around
    assert np.array_equal(O.scan_cpu(x), O.scan_cpu_loop(x))


@pytest.mark.parametrize("n", [1, 16384, 32768, (1 << 20) + 7])
def test_scan_matches_reference_cpu_loop(ref_cpu, n):
    # Inputs as the reference harness draws them: uniform 0..100 (evals/4090_scan/scan_harness.cuh:172).
    x = O.scan_inputs(n, seed=0xCA7CAFE, high=101)
    out = np.empty_like(x)
    ref_cpu.ref_scan_cpu(n, _ptr(x), _ptr(out))
    assert np.array_equal(O.scan_cpu(x), out)


def test_scan_wraparound_matches_reference_cpu_loop(ref_cpu):
    x = O.scan_inputs(100003, seed=3, high=0xFFFFFFFF)
    out = np.empty_like(x)
    ref_cpu.ref_scan_cpu(x.size, _ptr(x), _ptr(out))
    assert np.array_equal(O.scan_cpu(x), out)


def test_scan_c_restatement(oracle_c):
    x = O.scan_inputs(123457, seed=9, high=1 << 30)
    out = np.empty_like(x)
    oracle_c.oracle_scan_u32(x.size, _ptr(x), _ptr(out))
    assert np.array_equal(out, O.scan_cpu(x))


def test_scan_golden_fixture():
    """Fixture written by tests/golden/make_golden.py from the reference's scan_cpu."""
    g = np.load(GOLDEN / "scan_ref_cpu.npz")
    for key in ("small", "tile", "ragged", "wrap"):
        assert np.array_equal(O.scan_cpu(g[key + "_in"]), g[key + "_out"]), key


def test_sharded_scan_is_scan_of_concatenation():
    shards = [O.scan_inputs(n, seed=i, high=1 << 31) for i, n in enumerate([1000, 0, 4096, 17])]
    outs = O.sharded_scan_cpu(shards)
    carry = 0
    for s, o in zip(shards, outs):
        assert np.array_equal(o, (O.scan_cpu(s).astype(np.uint64) + carry).astype(np.uint32))
        carry = (carry + int(s.sum(dtype=np.uint64))) & 0xFFFFFFFF


def test_sgemm_c_restatement_within_tolerance(oracle_c):
    M, N, K = 96, 80, 200
    A, B, C = O.sgemm_inputs(M, N, K, seed=4)
    ref = O.sgemm_cpu(1.5, A, B, 0.5, C)
    out = C.copy()
    oracle_c.oracle_sgemm_f32(M, N, K, 1.5, _ptr(A), _ptr(B), 0.5, _ptr(out))
    assert O.sgemm_rel_error(out, ref) <= O.SGEMM_TOL


def test_sgemm_golden_fixture():
    """fp64 oracle against outputs of the reference's kernels 1-5 (recompiled for sm_100, run on a B200);
    fixture written by tests/golden/make_golden_gpu.py."""
    path = GOLDEN / "sgemm_ref_gpu.npz"
    if not path.exists():
        pytest.skip("GPU-generated fixture not present")
    g = np.load(path)
    ref = O.sgemm_cpu(float(g["alpha"]), g["A"], g["B"], float(g["beta"]), g["C"])
    for k in (1, 2, 3, 4, 5):
        assert O.sgemm_rel_error(g[f"out_k{k}"], ref) <= O.SGEMM_TOL, k


def test_bf16_rounding_matches_torch():
    import torch
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(100000).astype(np.float32) * 10.0 ** rng.integers(-20, 20, 100000),
                        np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.3895314e38], np.float32)]).astype(np.float32)
    bits = O.f32_to_bf16_bits(x)
    t = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(bits, t)
    assert np.array_equal(O.bf16_bits_to_f32(bits), torch.from_numpy(x).to(torch.bfloat16).float().numpy())


def test_gemm_bf16_c_restatement(oracle_c):
    M, N, K = 64, 48, 128
    A, B = O.gemm_bf16_inputs(M, N, K, seed=5)
    out = np.empty((N, M), np.uint16)
    oracle_c.oracle_gemm_bf16(M, N, K, _ptr(A), _ptr(B), _ptr(out))
    ok, worst = O.gemm_bf16_check(out, O.gemm_bf16_cpu(A, B))
    assert ok, worst


def test_gemm_bf16_layout_is_column_major_c():
    M, N, K = 8, 4, 16
    A, B = O.gemm_bf16_inputs(M, N, K, seed=6)
    ref = O.gemm_bf16_cpu(A, B)  # (N, M): element [n, m] sits at n * M + m
    a, b = O.bf16_bits_to_f32(A).astype(np.float64), O.bf16_bits_to_f32(B).astype(np.float64)
    assert ref.shape == (N, M)
    assert np.allclose(ref.ravel()[2 * M + 5], a[5] @ b[2])
