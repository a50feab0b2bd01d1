"""Host-buffer forms of the three operators: inputs and outputs live in (pinned)
host memory, device staging buffers are allocated once, and every call copies the
inputs to the device, runs the kernels through the C ABI and copies the result back.
This is what a caller with data in host memory uses, e.g. the reference harnesses,
which keep their matrices in host arrays and copy around each run
(evals/4090_scan/scan_harness.cuh:112-131, evals/h100_bench/main.cu:105-130).

The link to the host is the bottleneck of every one of them (the kernels take a tenth
of the copy time), so each call is cut into blocks along a dimension whose blocks are
contiguous on both sides, and three streams overlap the upload of block j+1, the
kernel on block j and the download of block j-1: uploads and downloads travel in
opposite directions of the link at the same time.  A call is asynchronous with respect
to the host like any other torch operation: it is ordered after the work already
queued on the current stream, and the current stream waits for it, so the caller
synchronises the current stream (or the device) before reading the host result.
"""
from __future__ import annotations

import torch

import prism_b200 as pb


def _blocks(n: int, block: int, quantum: int) -> list[tuple[int, int]]:
    """[lo, hi) ranges of about `block` items with boundaries on multiples of `quantum`; one range if n is small
    or not a multiple of the quantum."""
    if n <= 0:
        return []
    if n % quantum or n <= block:
        return [(0, n)]
    block = max(quantum, block // quantum * quantum)
    return [(lo, min(n, lo + block)) for lo in range(0, n, block)]


class _Lanes:
    """Upload, kernel and download streams, tied to the caller's current stream at both ends of a call."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.up = torch.cuda.Stream(self.device)
        self.run = torch.cuda.Stream(self.device)
        self.down = torch.cuda.Stream(self.device)

    def begin(self) -> None:
        cur = torch.cuda.current_stream(self.device)
        for s in (self.up, self.run, self.down):
            s.wait_stream(cur)

    def end(self) -> None:
        cur = torch.cuda.current_stream(self.device)
        for s in (self.up, self.run, self.down):
            cur.wait_stream(s)

    def stage(self, upload, kernel, download) -> None:
        """One block: `upload` on the upload stream, then `kernel`, then `download`, each on its own stream."""
        with torch.cuda.stream(self.up):
            upload()
            uploaded = self.up.record_event()
        with torch.cuda.stream(self.run):
            self.run.wait_event(uploaded)
            kernel()
            computed = self.run.record_event()
        with torch.cuda.stream(self.down):
            self.down.wait_event(computed)
            download()


class HostGemmBF16:
    """C (column-major M x N, i.e. an (N, M) tensor) = A @ B.T for host tensors.

    A is uploaded whole; B goes up in blocks of `block_rows` rows.  Rows of B are columns of the column-major
    C, i.e. contiguous row blocks of the (N, M) result, so each block's product can go back to the host while
    the next block of B is still arriving."""

    def __init__(self, M: int, N: int, K: int, device, block_rows: int = 1024):
        self.M, self.N, self.K = M, N, K
        self.a = torch.empty((M, K), dtype=torch.bfloat16, device=device)
        self.b = torch.empty((N, K), dtype=torch.bfloat16, device=device)
        self.c = torch.empty((N, M), dtype=torch.bfloat16, device=device)
        self.h2d_bytes = (M * K + N * K) * 2
        self.d2h_bytes = M * N * 2
        self.blocks = _blocks(N, block_rows, 256)
        self.lanes = _Lanes(device)

    def __call__(self, A_host: torch.Tensor, B_host: torch.Tensor, C_host: torch.Tensor) -> torch.Tensor:
        L = self.lanes
        L.begin()
        with torch.cuda.stream(L.up):
            self.a.copy_(A_host, non_blocking=True)
        for lo, hi in self.blocks:
            L.stage(lambda: self.b[lo:hi].copy_(B_host[lo:hi], non_blocking=True),
                    lambda: pb.runmyh100(self.M, hi - lo, self.K, self.a, self.b[lo:hi], self.c[lo:hi]),
                    lambda: C_host[lo:hi].copy_(self.c[lo:hi], non_blocking=True))
        L.end()
        return C_host


class HostSgemm:
    """C = alpha * A @ B + beta * C for host tensors (C is read and written).

    B is uploaded whole; A and C go up, and C comes back, in blocks of `block_rows` rows of M."""

    def __init__(self, M: int, N: int, K: int, device, kernel: int = 5, block_rows: int = 1024):
        self.M, self.N, self.K, self.kernel = M, N, K, kernel
        self.a = torch.empty((M, K), dtype=torch.float32, device=device)
        self.b = torch.empty((K, N), dtype=torch.float32, device=device)
        self.c = torch.empty((M, N), dtype=torch.float32, device=device)
        self.h2d_bytes = (M * K + K * N + M * N) * 4
        self.d2h_bytes = M * N * 4
        self.blocks = _blocks(M, block_rows, 128)
        self.lanes = _Lanes(device)

    def __call__(self, alpha, A_host, B_host, beta, C_host):
        L = self.lanes
        L.begin()
        with torch.cuda.stream(L.up):
            self.b.copy_(B_host, non_blocking=True)

        def upload(lo, hi):
            self.a[lo:hi].copy_(A_host[lo:hi], non_blocking=True)
            self.c[lo:hi].copy_(C_host[lo:hi], non_blocking=True)

        for lo, hi in self.blocks:
            L.stage(lambda: upload(lo, hi),
                    lambda: pb.run_my_kernel(self.kernel, hi - lo, self.N, self.K, alpha, self.a[lo:hi], self.b, beta,
                                             self.c[lo:hi]),
                    lambda: C_host[lo:hi].copy_(self.c[lo:hi], non_blocking=True))
        L.end()
        return C_host


class HostScan:
    """In-place inclusive scan of a host int32/uint32 tensor.

    The array goes through the device in blocks; each block is scanned starting from the last element of the
    block before it (kept on the device), so the blocks' results are final when they leave."""

    def __init__(self, n: int, device, block_elems: int | None = None):
        self.n = n
        self.x = torch.empty(n, dtype=torch.int32, device=device)
        if block_elems is None:
            block_elems = max(1 << 22, n // 16)
        self.blocks = _blocks(n, block_elems, 4)
        self.ws = pb.scan_workspace(max((hi - lo for lo, hi in self.blocks), default=0), device)
        self.carry = torch.zeros(1, dtype=torch.int32, device=device)
        self.h2d_bytes = n * 4
        self.d2h_bytes = n * 4
        self.lanes = _Lanes(device)

    def __call__(self, x_host: torch.Tensor) -> torch.Tensor:
        xh = x_host.view(torch.int32)
        L = self.lanes
        L.begin()
        with torch.cuda.stream(L.run):
            self.carry.zero_()

        def kernel(lo, hi):
            pb.scan_seeded_(self.x[lo:hi], self.ws, self.carry, 1)
            self.carry.copy_(self.x[hi - 1:hi])

        for lo, hi in self.blocks:
            L.stage(lambda: self.x[lo:hi].copy_(xh[lo:hi], non_blocking=True),
                    lambda: kernel(lo, hi),
                    lambda: xh[lo:hi].copy_(self.x[lo:hi], non_blocking=True))
        L.end()
        return x_host
