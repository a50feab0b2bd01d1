"""Host-buffer forms of the three operators: inputs and outputs live in (pinned)
host memory; every call copies the inputs to the device, runs the kernels and copies
the result back.  This is what a caller with data in host memory uses, e.g. the
reference harnesses, which keep their matrices in host arrays and copy around each run
(evals/4090_scan/scan_harness.cuh:112-131, evals/h100_bench/main.cu:105-130).

The classes are thin wrappers of the library's host plans (prism_b200_host_*_create /
_run / prism_b200_host_plan_destroy): the staging buffers, the three streams and the
block pipeline (upload of block j+1, kernel on block j and download of block j-1
overlap, the two copy directions running at once) live in the library, not here.  A call
is asynchronous like any other torch operation: it is ordered after the work already
queued on the current stream, and the current stream waits for it, so the caller
synchronises before reading the host result.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import load


def _host(name: str, t: torch.Tensor, dtypes, numel: int) -> None:
    if t.device.type != "cpu" or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous host tensor")
    if t.dtype not in dtypes:
        raise TypeError(f"{name} must have dtype in {dtypes}, got {t.dtype}")
    if t.numel() != numel:
        raise ValueError(f"{name} has {t.numel()} elements, the plan was made for {numel}")


class _Plan:
    def __init__(self, device):
        self.device = torch.device(device)
        self._plan = ctypes.c_void_p()

    def _stream(self) -> ctypes.c_void_p:
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    @property
    def blocks(self) -> int:
        """Number of blocks a call is cut into."""
        return int(load().prism_b200_host_plan_blocks(self._plan))

    def close(self) -> None:
        if self._plan:
            load().prism_b200_host_plan_destroy(self._plan)
            self._plan = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class HostGemmBF16(_Plan):
    """C (column-major M x N, i.e. an (N, M) tensor) = A @ B.T for host tensors."""

    def __init__(self, M: int, N: int, K: int, device, block_rows: int = 0):
        super().__init__(device)
        self.M, self.N, self.K = M, N, K
        self.h2d_bytes = (M * K + N * K) * 2
        self.d2h_bytes = M * N * 2
        with torch.cuda.device(self.device):
            _lib.check(load().prism_b200_host_gemm_bf16_create(M, N, K, int(block_rows), ctypes.byref(self._plan)))

    def __call__(self, A_host: torch.Tensor, B_host: torch.Tensor, C_host: torch.Tensor) -> torch.Tensor:
        _host("A", A_host, (torch.bfloat16,), self.M * self.K)
        _host("B", B_host, (torch.bfloat16,), self.N * self.K)
        _host("C", C_host, (torch.bfloat16,), self.N * self.M)
        with torch.cuda.device(self.device):
            _lib.check(load().prism_b200_host_gemm_bf16_run(self._plan, A_host.data_ptr(), B_host.data_ptr(),
                                                            C_host.data_ptr(), self._stream()))
        return C_host


class HostSgemm(_Plan):
    """C = alpha * A @ B + beta * C for host tensors (C is read and written)."""

    def __init__(self, M: int, N: int, K: int, device, kernel: int = 5, block_rows: int = 0):
        super().__init__(device)
        self.M, self.N, self.K, self.kernel = M, N, K, kernel
        self.h2d_bytes = (M * K + K * N + M * N) * 4
        self.d2h_bytes = M * N * 4
        with torch.cuda.device(self.device):
            _lib.check(load().prism_b200_host_sgemm_create(int(kernel), M, N, K, int(block_rows), ctypes.byref(self._plan)))

    def __call__(self, alpha, A_host, B_host, beta, C_host):
        _host("A", A_host, (torch.float32,), self.M * self.K)
        _host("B", B_host, (torch.float32,), self.K * self.N)
        _host("C", C_host, (torch.float32,), self.M * self.N)
        with torch.cuda.device(self.device):
            _lib.check(load().prism_b200_host_sgemm_run(self._plan, float(alpha), A_host.data_ptr(), B_host.data_ptr(),
                                                        float(beta), C_host.data_ptr(), self._stream()))
        return C_host


class HostScan(_Plan):
    """In-place inclusive scan of a host int32/uint32 tensor."""

    def __init__(self, n: int, device, block_elems: int = 0):
        super().__init__(device)
        self.n = n
        self.h2d_bytes = n * 4
        self.d2h_bytes = n * 4
        with torch.cuda.device(self.device):
            _lib.check(load().prism_b200_host_scan_create(int(n), int(block_elems or 0), ctypes.byref(self._plan)))

    def __call__(self, x_host: torch.Tensor) -> torch.Tensor:
        _host("x", x_host, (torch.int32, torch.uint32), self.n)
        with torch.cuda.device(self.device):
            _lib.check(load().prism_b200_host_scan_run(self._plan, x_host.data_ptr(), self._stream()))
        return x_host


# ---------------------------------------------------------------------------
# Pinned host memory on the GPU's own NUMA node
# ---------------------------------------------------------------------------
def _gpu_numa_cpus(device) -> set[int] | None:
    """CPUs of the NUMA node the GPU's PCIe link hangs off, from sysfs; None if the machine does not say."""
    try:
        p = torch.cuda.get_device_properties(device)
        bdf = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            text = f.read().strip()
        cpus: set[int] = set()
        for part in text.split(","):
            if "-" in part:
                lo, hi = part.split("-")
                cpus.update(range(int(lo), int(hi) + 1))
            elif part:
                cpus.add(int(part))
        return cpus or None
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None


def pinned_near(device, shape, dtype) -> torch.Tensor:
    """A pinned host tensor whose pages lie on the NUMA node of `device`'s PCIe link (where the machine exposes
    that): the allocating thread is confined to that node's CPUs while the pages are allocated and touched, then
    gets its CPU set back.  Several GPUs uploading at once then read from their own memory controllers instead of
    all from the node the process happened to start on.  Falls back to an ordinary pinned tensor."""
    import os
    cpus = _gpu_numa_cpus(device)
    old = None
    if cpus and hasattr(os, "sched_setaffinity"):
        try:
            old = os.sched_getaffinity(0)
            allowed = cpus & old
            if allowed:
                os.sched_setaffinity(0, allowed)
            else:
                old = None
        except OSError:
            old = None
    try:
        t = torch.empty(shape, dtype=dtype, pin_memory=True)
        t.view(torch.uint8).reshape(-1)[:: 4096].fill_(0)   # touch every page from this node
    finally:
        if old is not None:
            os.sched_setaffinity(0, old)
    return t
