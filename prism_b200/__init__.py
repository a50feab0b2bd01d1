"""prism_b200 -- B200 (sm_100a) kernels behind the entry points of the Prism
evaluation harnesses.

The functions named like the reference's launchers take the same arguments in
the same order and work in place on device memory:

    run_my_kernel(kernel_num, M, N, K, alpha, A, B, beta, C)   evals/4090_sgemm/runner.cu:245-267
    get_workspace_size(n), launch_scan(n, x, workspace)        evals/4090_scan/main.cu:63-86
    runmyh100(M, N, K, A, B, C)                                evals/h100_bench/utils.cuh:504-533

`sgemm`, `scan_` and `gemm_bf16` are thin conveniences over them that read the
sizes from the tensors.  Everything runs on the current CUDA stream of the
tensors' device through the C ABI in include/prism_b200.h; there is no CPU or
PyTorch fallback, and a missing library or a non-zero status raises.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import PrismB200Error, last_error, load  # noqa: F401

__all__ = [
    "run_my_kernel", "get_workspace_size", "launch_scan", "runmyh100",
    "sgemm", "scan_", "scan", "scan_f32_", "scan_static_", "scan_workspace", "gemm_bf16", "gemm_bf16_axpby", "reduce_u32", "scan_seeded_", "scan_add_carry_",
    "scan_publish_total", "scan_seeded_peers_", "scan_sharded_",
    "launch_count", "last_error", "clear_error", "version", "PrismB200Error",
]

_SCAN_DTYPES = (torch.int32, torch.uint32)


def _stream(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _require_cuda(name: str, t: torch.Tensor, dtype=None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError(f"{name} must be a CUDA tensor (prism_b200 has no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None:
        ok = t.dtype in dtype if isinstance(dtype, tuple) else t.dtype == dtype
        if not ok:
            raise TypeError(f"{name} has dtype {t.dtype}, expected {dtype}")


def version() -> int:
    return load().prism_b200_version()


def launch_count() -> int:
    """Kernels launched by the library since it was loaded."""
    return int(load().prism_b200_launch_count())


def clear_error() -> None:
    load().prism_b200_clear_error()


# ---------------------------------------------------------------------------
# FP32 SGEMM
# ---------------------------------------------------------------------------
def run_my_kernel(kernel_num: int, M: int, N: int, K: int, alpha: float, A: torch.Tensor, B: torch.Tensor,
                  beta: float, C: torch.Tensor) -> None:
    """C = alpha * A @ B + beta * C in place; row-major fp32; kernel_num 1..6."""
    for name, t, numel in (("A", A, M * K), ("B", B, K * N), ("C", C, M * N)):
        _require_cuda(name, t, torch.float32)
        if t.numel() < numel:
            raise ValueError(f"{name} holds {t.numel()} elements, needs {numel}")
    with torch.cuda.device(C.device):
        _lib.check(load().prism_b200_sgemm(int(kernel_num), int(M), int(N), int(K), float(alpha), A.data_ptr(),
                                           B.data_ptr(), float(beta), C.data_ptr(), _stream(C)))


def sgemm(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, alpha: float = 1.0, beta: float = 0.0,
          kernel: int = 5) -> torch.Tensor:
    if A.dim() != 2 or B.dim() != 2 or C.dim() != 2:
        raise ValueError("sgemm expects 2-D tensors")
    M, K = A.shape
    K2, N = B.shape
    if K2 != K or tuple(C.shape) != (M, N):
        raise ValueError(f"shape mismatch: A {tuple(A.shape)}, B {tuple(B.shape)}, C {tuple(C.shape)}")
    run_my_kernel(kernel, M, N, K, alpha, A, B, beta, C)
    return C


# ---------------------------------------------------------------------------
# uint32 inclusive scan
# ---------------------------------------------------------------------------
def get_workspace_size(n: int) -> int:
    out = ctypes.c_size_t(0)
    _lib.check(load().prism_b200_scan_workspace_size(int(n), ctypes.byref(out)))
    return int(out.value)


def scan_workspace(n: int, device) -> torch.Tensor:
    """Device scratch for a scan of n elements (contents do not matter)."""
    return torch.empty(get_workspace_size(n), dtype=torch.uint8, device=device)


def launch_scan(n: int, x: torch.Tensor, workspace: torch.Tensor) -> torch.Tensor:
    """In-place inclusive prefix sum of the first n elements of x (int32/uint32, wrap-around)."""
    _require_cuda("x", x, _SCAN_DTYPES)
    _require_cuda("workspace", workspace)
    if x.numel() < n:
        raise ValueError(f"x holds {x.numel()} elements, n = {n}")
    if workspace.numel() * workspace.element_size() < get_workspace_size(n):
        raise ValueError("workspace too small; see get_workspace_size(n)")
    with torch.cuda.device(x.device):
        _lib.check(load().prism_b200_scan(int(n), x.data_ptr(), workspace.data_ptr(), _stream(x)))
    return x


def scan_(x: torch.Tensor, workspace: torch.Tensor | None = None) -> torch.Tensor:
    n = x.numel()
    if workspace is None:
        workspace = scan_workspace(n, x.device)
    return launch_scan(n, x, workspace)


def scan_f32_(x: torch.Tensor, workspace: torch.Tensor | None = None) -> torch.Tensor:
    """In-place inclusive prefix sum of a float32 tensor (fp32 adds; last bits may vary between runs)."""
    _require_cuda("x", x, (torch.float32,))
    if workspace is None:
        workspace = scan_workspace(x.numel(), x.device)
    _require_cuda("workspace", workspace)
    if workspace.numel() * workspace.element_size() < get_workspace_size(x.numel()):
        raise ValueError("workspace too small; see get_workspace_size(n)")
    with torch.cuda.device(x.device):
        _lib.check(load().prism_b200_scan_f32(x.numel(), x.data_ptr(), workspace.data_ptr(), _stream(x)))
    return x


def scan(x: torch.Tensor, out: torch.Tensor | None = None, exclusive: bool = False,
         workspace: torch.Tensor | None = None) -> torch.Tensor:
    """Prefix sum of an int32/uint32, float32 or int64/uint64 tensor into `out` (a new tensor by default; `out`
    may be `x`).  Integer adds wrap around.  exclusive=True gives out[i] = x[0] + ... + x[i-1] with out[0] = 0."""
    _require_cuda("x", x, _SCAN_DTYPES + (torch.float32, torch.int64, torch.uint64))
    if out is None:
        out = torch.empty_like(x)
    _require_cuda("out", out, (x.dtype,))
    if out.numel() != x.numel() or out.device != x.device:
        raise ValueError("out must have the size and device of x")
    flags = (1 if exclusive else 0) | (2 if x.dtype == torch.float32 else 0) | (4 if x.element_size() == 8 else 0)
    need = ctypes.c_size_t(0)
    _lib.check(load().prism_b200_scan_general_workspace_size(x.numel(), flags, ctypes.byref(need)))
    if workspace is None:
        workspace = torch.empty(need.value, dtype=torch.uint8, device=x.device)
    _require_cuda("workspace", workspace)
    if workspace.numel() * workspace.element_size() < need.value:
        raise ValueError("workspace too small; see prism_b200_scan_general_workspace_size")
    with torch.cuda.device(x.device):
        _lib.check(load().prism_b200_scan_general(x.numel(), x.data_ptr(), out.data_ptr(), workspace.data_ptr(), flags,
                                                  _stream(x)))
    return out


def scan_static_(x: torch.Tensor) -> torch.Tensor:
    """In-place scan that allocates nothing: the look-back records live in a fixed array inside the
    library (at most 2^28 elements; calls that overlap on the GPU race -- see include/prism_b200.h)."""
    _require_cuda("x", x, _SCAN_DTYPES)
    with torch.cuda.device(x.device):
        _lib.check(load().prism_b200_scan_static(x.numel(), x.data_ptr(), _stream(x)))
    return x


def reduce_u32(x: torch.Tensor, total: torch.Tensor) -> torch.Tensor:
    """total[0] = wrap-around sum of x (device side, asynchronous)."""
    _require_cuda("x", x, _SCAN_DTYPES)
    _require_cuda("total", total, _SCAN_DTYPES)
    with torch.cuda.device(x.device):
        _lib.check(load().prism_b200_reduce_u32(x.numel(), x.data_ptr(), total.data_ptr(), _stream(x)))
    return total


def scan_seeded_(x: torch.Tensor, workspace: torch.Tensor, totals: torch.Tensor, rank: int) -> torch.Tensor:
    """Scan a shard in place starting from totals[0] + ... + totals[rank-1]."""
    _require_cuda("x", x, _SCAN_DTYPES)
    _require_cuda("workspace", workspace)
    _require_cuda("totals", totals, _SCAN_DTYPES)
    if totals.numel() < rank:
        raise ValueError("totals shorter than rank")
    if workspace.numel() * workspace.element_size() < get_workspace_size(x.numel()):
        raise ValueError("workspace too small; see get_workspace_size(n)")
    with torch.cuda.device(x.device):
        _lib.check(load().prism_b200_scan_seeded(x.numel(), x.data_ptr(), workspace.data_ptr(), totals.data_ptr(),
                                                 int(rank), _stream(x)))
    return x


def scan_publish_total(total: torch.Tensor, peer_slots_dev: int, world: int, rank: int, epoch: int) -> None:
    """Store {epoch, total[0]} into every rank's slot array.  `peer_slots_dev` is the device address of an
    array of `world` base addresses (e.g. `buffer_ptrs_dev` of a torch symmetric-memory handle)."""
    _require_cuda("total", total, _SCAN_DTYPES)
    with torch.cuda.device(total.device):
        _lib.check(load().prism_b200_scan_publish_total(total.data_ptr(), ctypes.c_void_p(int(peer_slots_dev)),
                                                        int(world), int(rank), int(epoch), _stream(total)))


def scan_seeded_peers_(x: torch.Tensor, workspace: torch.Tensor, slots: torch.Tensor, rank: int, world: int,
                       epoch: int) -> torch.Tensor:
    """Scan a shard in place; its first tile waits for all ranks' {epoch, total} words in `slots`
    (2 * world int64 words in this GPU's memory, written by the peers) and starts from the lower ranks' sum."""
    _require_cuda("x", x, _SCAN_DTYPES)
    _require_cuda("workspace", workspace)
    _require_cuda("slots", slots, torch.int64)
    if slots.numel() < 2 * world:
        raise ValueError("slots must hold 2 * world words")
    if workspace.numel() * workspace.element_size() < get_workspace_size(x.numel()):
        raise ValueError("workspace too small; see get_workspace_size(n)")
    with torch.cuda.device(x.device):
        _lib.check(load().prism_b200_scan_seeded_peers(x.numel(), x.data_ptr(), workspace.data_ptr(), slots.data_ptr(),
                                                       int(rank), int(world), int(epoch), _stream(x)))
    return x


def scan_sharded_(x: torch.Tensor, workspace: torch.Tensor, slots: torch.Tensor, peer_slots_dev: int, rank: int,
                  world: int, epoch: int, phases: int = 3, wait_limit_s: float = 0.0) -> torch.Tensor:
    """One launch of the sharded scan over peer memory: reduce the chunk and store its {epoch, total} word into
    every rank's `slots` (phases & 1), scan it in place starting from the lower ranks' totals (phases & 2).
    `wait_limit_s` bounds the wait for the other ranks' words (0 = the library's default of 1 s).  An empty
    chunk is allowed: it still publishes and waits."""
    _require_cuda("x", x, _SCAN_DTYPES)
    _require_cuda("workspace", workspace)
    _require_cuda("slots", slots, torch.int64)
    if slots.numel() < 2 * world:
        raise ValueError("slots must hold 2 * world words")
    if workspace.numel() * workspace.element_size() < get_workspace_size(x.numel()):
        raise ValueError("workspace too small; see get_workspace_size(n)")
    with torch.cuda.device(x.device):
        _lib.check(load().prism_b200_scan_sharded(x.numel(), x.data_ptr() if x.numel() else None, workspace.data_ptr(),
                                                  slots.data_ptr(), ctypes.c_void_p(int(peer_slots_dev)), int(rank),
                                                  int(world), int(epoch), int(phases), int(wait_limit_s * 1e9), _stream(x)))
    return x


def scan_add_carry_(x: torch.Tensor, totals: torch.Tensor, rank: int) -> torch.Tensor:
    """x += totals[0] + ... + totals[rank-1] (second pass of the two-pass sharded scan)."""
    _require_cuda("x", x, _SCAN_DTYPES)
    _require_cuda("totals", totals, _SCAN_DTYPES)
    if totals.numel() < rank:
        raise ValueError("totals shorter than rank")
    with torch.cuda.device(x.device):
        _lib.check(load().prism_b200_scan_add_carry(x.numel(), x.data_ptr(), totals.data_ptr(), int(rank),
                                                    _stream(x)))
    return x


# ---------------------------------------------------------------------------
# bf16 GEMM, C = A @ B.T, C column-major
# ---------------------------------------------------------------------------
def runmyh100(M: int, N: int, K: int, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor) -> None:
    """A: M x K, B: N x K (both K-major bf16); C: M x N bf16 written column-major (C[n * M + m])."""
    for name, t, numel in (("A", A, M * K), ("B", B, N * K), ("C", C, M * N)):
        _require_cuda(name, t, torch.bfloat16)
        if t.numel() < numel:
            raise ValueError(f"{name} holds {t.numel()} elements, needs {numel}")
    with torch.cuda.device(C.device):
        _lib.check(load().prism_b200_gemm_bf16(int(M), int(N), int(K), A.data_ptr(), B.data_ptr(), C.data_ptr(),
                                               _stream(C)))


def gemm_bf16_axpby(alpha: float, A: torch.Tensor, B: torch.Tensor, beta: float, C: torch.Tensor,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """alpha * (A @ B.T) + beta * C for A (M, K), B (N, K) and C given as the (N, M) tensor that holds the
    column-major M x N matrix; returns `out` in the same layout (C itself by default: in place)."""
    M, K = A.shape
    N, K2 = B.shape
    if K2 != K:
        raise ValueError(f"K mismatch: A {tuple(A.shape)}, B {tuple(B.shape)}")
    if out is None:
        out = C
    for name, t, numel in (("A", A, M * K), ("B", B, N * K), ("C", C, M * N), ("out", out, M * N)):
        _require_cuda(name, t, torch.bfloat16)
        if t.numel() != numel:
            raise ValueError(f"{name} holds {t.numel()} elements, needs {numel}")
    with torch.cuda.device(out.device):
        _lib.check(load().prism_b200_gemm_bf16_axpby(int(M), int(N), int(K), float(alpha), A.data_ptr(), B.data_ptr(),
                                                     float(beta), C.data_ptr(), out.data_ptr(), _stream(out)))
    return out


def gemm_bf16(A: torch.Tensor, B: torch.Tensor, out: torch.Tensor | None = None, row_major: bool = False) -> torch.Tensor:
    """A @ B.T for A (M, K) and B (N, K), bf16 with fp32 accumulation.

    By default returns C^T as an (N, M) row-major tensor, i.e. the reference's column-major M x N C
    (`out.t()` is the product).  row_major=True returns the (M, N) row-major product itself: the same
    kernel with the two operands exchanged.
    """
    M, K = A.shape
    N, K2 = B.shape
    if K2 != K:
        raise ValueError(f"K mismatch: A {tuple(A.shape)}, B {tuple(B.shape)}")
    if row_major:
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
        runmyh100(N, M, K, B, A, out)
        return out
    if out is None:
        out = torch.empty((N, M), dtype=torch.bfloat16, device=A.device)
    runmyh100(M, N, K, A, B, out)
    return out
