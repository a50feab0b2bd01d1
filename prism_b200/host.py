"""Host-buffer forms of the three operators: inputs and outputs live in (pinned)
host memory, device staging buffers are allocated once, and every call copies the
inputs to the device, runs the kernel through the C ABI and copies the result back,
all on the current stream.  This is what a caller with data in host memory uses,
e.g. the reference harnesses, which keep their matrices in host arrays and copy
around each run (evals/4090_scan/scan_harness.cuh:112-131, evals/h100_bench/main.cu:105-130).
"""
from __future__ import annotations

import torch

import prism_b200 as pb


class HostGemmBF16:
    """C (column-major M x N, i.e. an (N, M) tensor) = A @ B.T for host tensors."""

    def __init__(self, M: int, N: int, K: int, device):
        self.M, self.N, self.K = M, N, K
        self.a = torch.empty((M, K), dtype=torch.bfloat16, device=device)
        self.b = torch.empty((N, K), dtype=torch.bfloat16, device=device)
        self.c = torch.empty((N, M), dtype=torch.bfloat16, device=device)
        self.h2d_bytes = (M * K + N * K) * 2
        self.d2h_bytes = M * N * 2

    def __call__(self, A_host: torch.Tensor, B_host: torch.Tensor, C_host: torch.Tensor) -> torch.Tensor:
        self.a.copy_(A_host, non_blocking=True)
        self.b.copy_(B_host, non_blocking=True)
        pb.runmyh100(self.M, self.N, self.K, self.a, self.b, self.c)
        C_host.copy_(self.c, non_blocking=True)
        return C_host


class HostSgemm:
    """C = alpha * A @ B + beta * C for host tensors (C is read and written)."""

    def __init__(self, M: int, N: int, K: int, device, kernel: int = 5):
        self.M, self.N, self.K, self.kernel = M, N, K, kernel
        self.a = torch.empty((M, K), dtype=torch.float32, device=device)
        self.b = torch.empty((K, N), dtype=torch.float32, device=device)
        self.c = torch.empty((M, N), dtype=torch.float32, device=device)
        self.h2d_bytes = (M * K + K * N + M * N) * 4
        self.d2h_bytes = M * N * 4

    def __call__(self, alpha, A_host, B_host, beta, C_host):
        self.a.copy_(A_host, non_blocking=True)
        self.b.copy_(B_host, non_blocking=True)
        self.c.copy_(C_host, non_blocking=True)
        pb.run_my_kernel(self.kernel, self.M, self.N, self.K, alpha, self.a, self.b, beta, self.c)
        C_host.copy_(self.c, non_blocking=True)
        return C_host


class HostScan:
    """In-place inclusive scan of a host int32/uint32 tensor."""

    def __init__(self, n: int, device):
        self.n = n
        self.x = torch.empty(n, dtype=torch.int32, device=device)
        self.ws = pb.scan_workspace(n, device)
        self.h2d_bytes = n * 4
        self.d2h_bytes = n * 4

    def __call__(self, x_host: torch.Tensor) -> torch.Tensor:
        self.x.copy_(x_host.view(torch.int32), non_blocking=True)
        pb.launch_scan(self.n, self.x, self.ws)
        x_host.view(torch.int32).copy_(self.x, non_blocking=True)
        return x_host
