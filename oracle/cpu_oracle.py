"""CPU oracle for the three kernel families -- TEST INFRASTRUCTURE ONLY.

Nothing in the `prism_b200` package imports this module; it is the checker used
by `tests/`, by `__graft_entry__.smoke()` and by the CPU-baseline legs of
`bench.py`.  It restates in NumPy what the reference's kernels compute, and
provides the seeded input generators of the benchmark configurations.

Parity status (what pins each restatement):
  * scan   -- pinned.  `scan_cpu` below is checked against the reference's own CPU
              loop `scan_cpu` (evals/4090_scan/scan_harness.cuh:30-36), compiled
              from where it lies into oracle/_ref/ by oracle/build_ref.py, and against
              the committed fixture tests/golden/scan_ref_cpu.npz produced by it; on
              a GPU also against the reference `scan_kernel` recompiled for sm_100.
  * sgemm  -- the reference has no CPU implementation and no golden vectors for
              this path (its harness compares with cuBLAS, evals/4090_sgemm/runner.cu:105-117).
              The restatement is fp64 NumPy, as the benchmark definition prescribes;
              it is pinned on a GPU against the reference kernels 1, 2, 3, 4, 5 recompiled
              for sm_100 (oracle/_ref) and against fixtures generated from them.
  * bf16   -- PARITY UNPINNED by the reference: its kernel is wgmma/sm_90a-only and
              cannot run on sm_100, it has no CPU implementation and no golden
              vectors (its harness compares with cuBLAS, evals/h100_bench/main.cu:43-55,116-136).
              The restatement is fp64 NumPy on the bf16-rounded inputs.
"""
from __future__ import annotations

import numpy as np

# ---------------------------------------------------------------------------
# scan
# ---------------------------------------------------------------------------


def scan_cpu(x: np.ndarray) -> np.ndarray:
    """Inclusive prefix sum with 32-bit wrap-around.

    Follows `scan_cpu` (evals/4090_scan/scan_harness.cuh:30-36): a running
    uint32 accumulator, out[i] = acc after adding x[i].  np.cumsum with a uint32
    accumulator is the same arithmetic (addition modulo 2^32 is associative).
    """
    x = np.ascontiguousarray(x).view(np.uint32)
    return np.cumsum(x, dtype=np.uint32)


def scan_f32_cpu(x: np.ndarray) -> np.ndarray:
    """fp64 running sum of float32 values: the value an fp32 scan approximates.  The reference has no
    floating-point scan (its kernel and its CPU loop are uint32, evals/4090_scan/scan_harness.cuh:30-36);
    this is the checker of the library's fp32 flavour, compared with a tolerance."""
    return np.cumsum(np.ascontiguousarray(x, dtype=np.float32).astype(np.float64))


def scan_i64_cpu(x: np.ndarray) -> np.ndarray:
    """Inclusive prefix sum of 64-bit integers with wrap-around: the reference's loop
    (evals/4090_scan/scan_harness.cuh:30-36) with a 64-bit accumulator.  The reference scans uint32 only; this
    is the checker of the library's 64-bit flavour."""
    return np.cumsum(np.ascontiguousarray(x).view(np.uint64), dtype=np.uint64)


def scan_cpu_loop(x: np.ndarray) -> np.ndarray:
    """The same thing as a literal loop (small inputs only); used to pin `scan_cpu`."""
    x = np.ascontiguousarray(x).view(np.uint32)
    out = np.empty_like(x)
    acc = 0
    for i in range(x.size):
        acc = (acc + int(x[i])) & 0xFFFFFFFF
        out[i] = acc
    return out


def scan_total_int64(x: np.ndarray) -> int:
    """Overflow-checked total (the int64 check of the 2^30 configuration)."""
    return int(np.sum(np.ascontiguousarray(x).view(np.uint32), dtype=np.int64))


def sharded_scan_cpu(shards: list[np.ndarray]) -> list[np.ndarray]:
    """What the sharded path must produce: the scan of the concatenation, cut back into shards."""
    full = scan_cpu(np.concatenate([np.ascontiguousarray(s).view(np.uint32) for s in shards]))
    out, pos = [], 0
    for s in shards:
        out.append(full[pos:pos + s.size])
        pos += s.size
    return out


# ---------------------------------------------------------------------------
# SGEMM
# ---------------------------------------------------------------------------


def sgemm_cpu(alpha: float, A: np.ndarray, B: np.ndarray, beta: float, C: np.ndarray) -> np.ndarray:
    """fp64 value of  alpha * A @ B + beta * C  (row-major), the quantity every
    reference SGEMM kernel approximates in fp32
    (generated/my_sgemm_kernel_1.cu:19-23 and the epilogues of kernels 2-5)."""
    return alpha * (A.astype(np.float64) @ B.astype(np.float64)) + beta * C.astype(np.float64)


def sgemm_rel_error(C_out: np.ndarray, C_ref64: np.ndarray) -> float:
    """Norm-wise relative error  max|C - C_ref| / max|C_ref|.

    With zero-mean inputs some outputs are arbitrarily close to zero, so an
    element-wise ratio has no bound even for a correctly rounded kernel; the
    benchmark's 1e-5 bound is applied to this quantity."""
    denom = float(np.max(np.abs(C_ref64)))
    if denom == 0.0:
        denom = 1.0
    return float(np.max(np.abs(C_out.astype(np.float64) - C_ref64))) / denom


SGEMM_TOL = 1e-5

# ---------------------------------------------------------------------------
# bf16 GEMM
# ---------------------------------------------------------------------------


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16, returned as uint16 bit patterns."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    bias = np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))
    return ((b + bias) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def gemm_bf16_cpu(A_bits: np.ndarray, B_bits: np.ndarray) -> np.ndarray:
    """fp64 value of the reference bf16 kernel's output, in ITS memory layout.

    A is M x K, B is N x K (K contiguous); the kernel stores C[n * M + m]
    (generated/cutlass_my_h100_match_no_tail.cu:313,347-354), i.e. an (N, M)
    row-major array, which is what this returns (before the final bf16 rounding)."""
    A = bf16_bits_to_f32(A_bits).astype(np.float64)
    B = bf16_bits_to_f32(B_bits).astype(np.float64)
    return B @ A.T


def gemm_bf16_axpby_cpu(alpha: float, A_bits: np.ndarray, B_bits: np.ndarray, beta: float, C_bits: np.ndarray) -> np.ndarray:
    """fp64 value of alpha * (A @ B^T) + beta * C in the kernel's (N, M) layout; C_bits is the (N, M) array of bf16
    bit patterns.  The reference's bf16 kernel has no such epilogue (its SGEMM kernels do,
    generated/my_sgemm_kernel_5.cu:56-77); this is the checker of the library's flavour."""
    C = bf16_bits_to_f32(C_bits).astype(np.float64).reshape(B_bits.shape[0], A_bits.shape[0])
    return alpha * gemm_bf16_cpu(A_bits, B_bits) + beta * C


GEMM_BF16_RTOL = 1e-2


def gemm_bf16_check(C_bits: np.ndarray, ref64: np.ndarray) -> tuple[bool, float]:
    """|D - D_ref| <= 1e-2 * |D_ref| + 1e-2 * rms(D_ref), element-wise; returns (ok, worst ratio)."""
    got = bf16_bits_to_f32(C_bits).astype(np.float64).reshape(ref64.shape)
    rms = float(np.sqrt(np.mean(ref64 * ref64)))
    bound = GEMM_BF16_RTOL * np.abs(ref64) + GEMM_BF16_RTOL * rms
    ratio = np.abs(got - ref64) / np.maximum(bound, 1e-300)
    return bool(np.all(ratio <= 1.0)), float(np.max(ratio))


# ---------------------------------------------------------------------------
# Seeded inputs of the benchmark configurations
# ---------------------------------------------------------------------------


def sgemm_inputs(M: int, N: int, K: int, seed: int, zero_c: bool = False):
    """A, B (and C) uniform[-1, 1) float32, row-major."""
    rng = np.random.default_rng(seed)
    A = rng.uniform(-1.0, 1.0, (M, K)).astype(np.float32)
    B = rng.uniform(-1.0, 1.0, (K, N)).astype(np.float32)
    C = np.zeros((M, N), np.float32) if zero_c else rng.uniform(-1.0, 1.0, (M, N)).astype(np.float32)
    return A, B, C


def gemm_bf16_inputs(M: int, N: int, K: int, seed: int):
    """A (M x K), B (N x K) = 0.1 * normal(0, 1) rounded to bf16; uint16 bit patterns."""
    rng = np.random.default_rng(seed)
    A = f32_to_bf16_bits((0.1 * rng.standard_normal((M, K))).astype(np.float32))
    B = f32_to_bf16_bits((0.1 * rng.standard_normal((N, K))).astype(np.float32))
    return A, B


def scan_inputs(n: int, seed: int, high: int = 16) -> np.ndarray:
    """uint32 values uniform in [0, high)."""
    rng = np.random.default_rng(seed)
    return rng.integers(0, high, n, dtype=np.uint32)
