"""Multi-GPU forms of the two paths that shard: one process per GPU.

* GEMM (fp32 and bf16): rows of M are independent given all of B.  Rank r owns
  rows [r * M / g, (r + 1) * M / g) of A and of C; B is replicated.  There is no
  collective on the data path.
* scan: rank r owns the r-th contiguous chunk.  The only exchange is one uint32
  total per rank.  Three schedules are offered:
    "peer_words"        ONE launch per rank: the CTAs add up the chunk (4 B/element read) and the
                        total is stored as an {epoch, total} word straight into every rank's memory
                        over NVLink (symmetric memory, no collective call, no host involvement);
                        then the scan, whose first tile waits for the words and starts from the sum
                        of the lower ranks' totals (8 B/element): 12 B/element per rank.  Default on
                        CUDA with more than one rank; if the symmetric-memory rendezvous is not
                        available (no peer access, several nodes) the constructor falls back to
                        "reduce_then_scan".  The wait for the other ranks is bounded
                        (`wait_limit_s`): ranks that enter the call further apart than that get a
                        device time-out instead of a result -- `checked=True` makes the call
                        synchronise and raise in that case; otherwise consult `last_error()` after
                        synchronising.
    "reduce_then_scan"  the same in two launches with an NCCL all-gather of the totals in between
                        (waits as long as NCCL does).
    "scan_then_carry"   local scan (8 B/element), all-gather of the last elements,
                        carry-add pass (8 B/element): 16 B/element per rank.
  All produce the scan of the concatenated array, bit for bit.

The reference has no multi-GPU code; its scan harness works on one device
(evals/4090_scan/main.cu:96-128).
"""
from __future__ import annotations

import ctypes
from typing import Any

import torch
import torch.distributed as dist


def chunk_bounds(n: int, world: int, rank: int, align: int = 4) -> tuple[int, int]:
    """Contiguous chunk [lo, hi) of rank `rank`; interior boundaries are multiples of `align`
    (16-byte alignment of every shard start for uint32 data)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    per = -(-n // world)            # ceil
    per = -(-per // align) * align  # round up to the alignment
    lo = min(n, rank * per)
    hi = min(n, (rank + 1) * per)
    return lo, hi


def head_tail_bounds(n: int, world: int, align: int = 8) -> tuple[int, int, int] | None:
    """Sizes (head, chunk, tail) of the head_tail schedule, or None where n is too small for it.

    Rank 0 owns the first `head` = chunk / 2 elements and the last `tail` <= chunk elements of the array, rank
    r >= 1 the chunk [head + (r - 1) chunk, head + r chunk).  Rank 0 moves 8 bytes per element (its head needs no
    prefix, its tail's total is needed by nobody), the others 12 (add up, then scan), so 1.5 chunks on rank 0 take as
    long as one chunk elsewhere: n = (world + 0.5) chunk.  All piece boundaries are multiples of `align` / 2 elements."""
    if world < 2:
        return None
    chunk = -(-2 * n // (2 * world + 1))          # ceil(n / (world + 0.5))
    chunk = -(-chunk // align) * align
    head = chunk // 2
    tail = n - head - (world - 1) * chunk
    if chunk == 0 or tail < 0:
        return None
    return head, chunk, tail


def head_tail_pieces(n: int, world: int, rank: int) -> list[tuple[int, int]]:
    """The [lo, hi) ranges of the array that `rank` owns under the head_tail schedule, in the order they lie in its
    local buffer (rank 0: head, then tail)."""
    b = head_tail_bounds(n, world)
    if b is None:
        raise ValueError(f"n = {n} is too small for the head_tail schedule on {world} ranks")
    head, chunk, tail = b
    if rank == 0:
        return [(0, head), (n - tail, n)]
    return [(head + (rank - 1) * chunk, head + rank * chunk)]


def row_shard(M: int, world: int, rank: int, tile: int = 128) -> tuple[int, int]:
    """Rows [lo, hi) of A and C owned by `rank`; M / world must be a multiple of the M tile."""
    if M % world or (M // world) % tile:
        raise ValueError(f"M={M} does not split into {world} shards of a multiple of {tile} rows")
    per = M // world
    return rank * per, (rank + 1) * per


class _CudaOps:
    """The real kernels (C ABI).  Tests on CPU pass a stand-in with the same four methods."""

    def __init__(self):
        import prism_b200 as pb
        self._pb = pb

    def workspace(self, n, device):
        return self._pb.scan_workspace(n, device)

    def reduce_u32(self, x, total):
        self._pb.reduce_u32(x, total)

    def scan_seeded_(self, x, workspace, totals, rank):
        self._pb.scan_seeded_(x, workspace, totals, rank)

    def scan_(self, x, workspace):
        self._pb.launch_scan(x.numel(), x, workspace)

    def scan_add_carry_(self, x, totals, rank):
        self._pb.scan_add_carry_(x, totals, rank)

    def scan_sharded_(self, x, workspace, slots, peer_slots_dev, rank, world, epoch, wait_limit_s):
        self._pb.scan_sharded_(x, workspace, slots, peer_slots_dev, rank, world, epoch, 3, wait_limit_s)

    def scan_head_tail_(self, head, tail, ws_head, ws_tail, zero, slots, peer_slots_dev, world, epoch, wait_limit_s):
        """Rank 0 of the head_tail schedule: scan the head, publish its total (its last element, or `zero` for an
        empty head), then scan the tail from the sum of all the ranks' totals."""
        if head.numel():
            self._pb.launch_scan(head.numel(), head, ws_head)
        self._pb.scan_publish_total(head[-1:] if head.numel() else zero, peer_slots_dev, world, 0, epoch)
        self._pb.scan_sharded_(tail, ws_tail, slots, peer_slots_dev, world, world, epoch, 2, wait_limit_s)

    def check(self, device):
        """Synchronise and raise if a device-side wait ran out."""
        import torch as _t
        _t.cuda.synchronize(device)
        code, msg = self._pb.last_error()
        if code:
            self._pb.clear_error()
            raise self._pb.PrismB200Error(code, msg)


def _symmetric_bytes(n_bytes: int, device, group):
    """`n_bytes` of device memory on this rank that every rank of the group can write (uint8 tensor), the
    symmetric-memory handle, and the list of all ranks' base addresses; None if torch's symmetric memory cannot
    provide them."""
    try:
        import torch.distributed._symmetric_memory as symm
        raw = symm.empty(n_bytes, dtype=torch.uint8, device=device)
        handle = symm.rendezvous(raw, group if group is not None else dist.group.WORLD)
        return raw, handle, [int(p) for p in handle.buffer_ptrs]
    except Exception as e:   # no peer access, several nodes, or a torch build without the module
        import warnings
        warnings.warn(f"peer exchange unavailable ({type(e).__name__}: {e}); using NCCL all-gathers")
        return None


def _symmetric_words(n_words: int, device, group):
    """`n_words` int64 words on this rank that every rank of the group can write, plus the device address of
    the table of all ranks' base addresses; None if torch's symmetric memory cannot provide them."""
    try:
        import torch.distributed._symmetric_memory as symm
        words = symm.empty(n_words, dtype=torch.int64, device=device)
        words.zero_()
        handle = symm.rendezvous(words, group if group is not None else dist.group.WORLD)
        return words, handle, int(handle.buffer_ptrs_dev)
    except Exception as e:   # no peer access, several nodes, or a torch build without the module
        import warnings
        warnings.warn(f"peer_words schedule unavailable ({type(e).__name__}: {e}); using reduce_then_scan")
        return None


class ShardedScan:
    """In-place inclusive scan of an array cut into one contiguous chunk per rank."""

    SCHEDULES = ("reduce_then_scan", "scan_then_carry")       # run anywhere a process group runs
    PEER_SCHEDULE = "peer_words"                               # needs CUDA peer access (one node)
    HEAD_TAIL = "head_tail"    # peer_words with rank 0 owning a head and a tail of the array: see head_tail_bounds

    def __init__(self, n_local: int, device, group: Any = None, schedule: str | None = None, ops: Any = None,
                 wait_limit_s: float = 0.0, checked: bool = False, symmetric_words: Any = _symmetric_words, head: int = 0):
        """`head` (head_tail schedule, rank 0 only): how many of the n_local elements are the head of the array; the
        rest of the local buffer is its tail.  Without peer-writable words head_tail cannot run and raises."""
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        on_cuda = torch.device(device).type == "cuda"
        asked = schedule
        if schedule is None:
            schedule = self.PEER_SCHEDULE if (on_cuda and self.world > 1 and ops is None) else "reduce_then_scan"
        self.head_tail = schedule == self.HEAD_TAIL
        if self.head_tail:
            if self.world < 2:
                raise ValueError("the head_tail schedule needs at least two ranks")
            schedule = self.PEER_SCHEDULE        # the same words, the same kernels; rank 0 runs them differently
        if schedule not in self.SCHEDULES + (self.PEER_SCHEDULE,):
            raise ValueError(f"schedule must be one of {self.SCHEDULES + (self.PEER_SCHEDULE, self.HEAD_TAIL)}")
        if schedule == self.PEER_SCHEDULE and self.world > 32:
            raise ValueError("the peer_words schedule handles at most 32 ranks")
        if schedule == self.PEER_SCHEDULE and not on_cuda and ops is None:
            raise ValueError("the peer_words schedule needs CUDA devices")
        self.epoch = 0
        self.slots = None
        self.peer_slots_dev = 0
        self.wait_limit_s = float(wait_limit_s)
        self.checked = bool(checked)
        self.device = device
        self.ops = ops if ops is not None else _CudaOps()
        self.n_local = n_local
        self.head = int(head) if (self.head_tail and self.rank == 0) else 0
        if not 0 <= self.head <= n_local or self.head % 4:
            raise ValueError("head must lie within the local buffer and be a multiple of 4 elements")
        self.workspace = self.ops.workspace(n_local, device)
        self.workspace_head = self.ops.workspace(self.head, device) if self.head_tail and self.rank == 0 else None
        self.total = torch.zeros(1, dtype=torch.int32, device=device)
        self.totals = torch.zeros(self.world, dtype=torch.int32, device=device)
        if schedule == self.PEER_SCHEDULE and self.world > 1:
            # 2 * world words per rank, writable by every rank.  All ranks must agree on the outcome,
            # hence the all-reduce of "it worked here".
            got = symmetric_words(2 * self.world, device, group)
            ok = torch.tensor([1 if got is not None else 0], dtype=torch.int32, device=device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok.item()) == 1:
                self.slots, self._symm, self.peer_slots_dev = got
                if on_cuda:
                    torch.cuda.synchronize(device)
                dist.barrier(group)   # every rank's words are zero before anyone publishes
            elif self.head_tail:
                raise RuntimeError("the head_tail schedule needs peer-writable words (one node with peer access)")
            else:
                schedule = "reduce_then_scan"
        elif schedule == self.PEER_SCHEDULE and on_cuda and ops is None and asked == self.PEER_SCHEDULE:
            # One rank, asked for by name: the same kernel with this rank as its only peer (12 B/element instead of
            # the plain scan's 8).  Of no use in production; it lets the sharded kernel be measured on one GPU.
            self.slots = torch.zeros(2, dtype=torch.int64, device=device)
            self._table = torch.tensor([self.slots.data_ptr()], dtype=torch.int64, device=device)
            self.peer_slots_dev = int(self._table.data_ptr())
        self.schedule = self.HEAD_TAIL if self.head_tail else schedule
        self.fell_back = asked in (None, self.PEER_SCHEDULE) and schedule != self.PEER_SCHEDULE and on_cuda and self.world > 1

    def _exchange(self, total: torch.Tensor) -> None:
        if self.world == 1:
            self.totals.copy_(total)
        else:
            dist.all_gather_into_tensor(self.totals, total, group=self.group)

    def __call__(self, x_local: torch.Tensor) -> torch.Tensor:
        if x_local.numel() != self.n_local:
            raise ValueError(f"shard has {x_local.numel()} elements, planned for {self.n_local}")
        if self.head_tail and self.rank == 0:
            self.epoch += 1
            self.ops.scan_head_tail_(x_local[:self.head], x_local[self.head:], self.workspace_head, self.workspace,
                                     self.total.zero_(), self.slots, self.peer_slots_dev, self.world, self.epoch,
                                     self.wait_limit_s)
            if self.checked:
                self.ops.check(self.device)
        elif self.schedule in (self.PEER_SCHEDULE, self.HEAD_TAIL) and self.slots is not None:
            self.epoch += 1
            self.ops.scan_sharded_(x_local, self.workspace, self.slots, self.peer_slots_dev, self.rank, self.world,
                                   self.epoch, self.wait_limit_s)
            if self.checked:
                self.ops.check(self.device)
        elif self.schedule in ("reduce_then_scan", self.PEER_SCHEDULE):
            if self.world > 1:
                self.ops.reduce_u32(x_local, self.total)
                self._exchange(self.total)
            self.ops.scan_seeded_(x_local, self.workspace, self.totals, self.rank)
        else:
            self.ops.scan_(x_local, self.workspace)
            if self.world > 1:
                # After a local inclusive scan the last element is the chunk total.
                last = x_local[-1:] if self.n_local else self.total.zero_()
                self._exchange(last.view(torch.int32) if last.dtype != torch.int32 else last)
                self.ops.scan_add_carry_(x_local, self.totals, self.rank)
        return x_local

    def totals_int64(self) -> list[int]:
        """Per-rank totals of the last call as non-negative Python ints (for the host-side overflow check)."""
        if self.slots is not None and self.epoch > 0:
            half = self.slots.cpu().tolist()[(self.epoch & 1) * self.world:][: self.world]
            return [(int(w) >> 32) & 0xFFFFFFFF for w in half]
        return [int(v) & 0xFFFFFFFF for v in self.totals.cpu().tolist()]


class RowShardedGemmBF16:
    """C = A @ B.T with A and C cut by rows of M; each rank computes its own rows, no collective.

    The rank's C shard is its own column-major (M / g) x N buffer, i.e. an (N, M / g)
    row-major tensor, as the single-GPU kernel writes it.
    """

    def __init__(self, M: int, N: int, K: int, group: Any = None):
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.lo, self.hi = row_shard(M, self.world, self.rank)
        self.M, self.N, self.K = M, N, K

    @property
    def rows(self) -> int:
        return self.hi - self.lo

    def __call__(self, A_local: torch.Tensor, B: torch.Tensor, C_local: torch.Tensor) -> torch.Tensor:
        import prism_b200 as pb
        pb.runmyh100(self.rows, self.N, self.K, A_local, B, C_local)
        return C_local


class RowShardedSgemm:
    """C = alpha * A @ B + beta * C with A and C cut by rows of M; no collective."""

    def __init__(self, M: int, N: int, K: int, group: Any = None, kernel: int = 5):
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.lo, self.hi = row_shard(M, self.world, self.rank)
        self.M, self.N, self.K, self.kernel = M, N, K, kernel

    @property
    def rows(self) -> int:
        return self.hi - self.lo

    def __call__(self, alpha: float, A_local: torch.Tensor, B: torch.Tensor, beta: float,
                 C_local: torch.Tensor) -> torch.Tensor:
        import prism_b200 as pb
        pb.run_my_kernel(self.kernel, self.rows, self.N, self.K, alpha, A_local, B, beta, C_local)
        return C_local


class ShardedHostGemmBF16:
    """C = A @ B.T for operands in HOST memory on g GPUs (one process each), rows of M sharded.

    Every rank holds its rows of A, all of B and its (N, M / g) block of the column-major C in pinned host
    memory.  B is the same on every rank, so no rank uploads all of it: per step each rank sends 1/g of a
    block of B's rows over its own PCIe link, the ranks complete the block over NVLink in their OWN memory, and
    the GEMM on that block of columns of C runs while the next block is uploaded and gathered and the previous
    block of C goes back to the host.  The exchange is one-sided by default (`exchange="peer"`): each rank pushes
    its piece into every other rank's copy of B with the library's own copy kernel and raises a flag there
    (prism_b200_peer_push), and the kernel stream waits, bounded, for all ranks' flags of the block
    (prism_b200_peer_wait) -- no collective call, nothing waits inside the copy.  B is double-buffered by the
    parity of the call, since a rank can be one call ahead of another.  `exchange="nccl"` does the same with an
    in-place NCCL all-gather per block and is what runs where symmetric memory is not available.  Either way the
    GEMM only ever reads local HBM:

        upload stream    piece 0 | A rows | piece 1 | piece 2 | ...
        gather stream             gather 0          | gather 1 | ...
        kernel stream                      GEMM 0            | GEMM 1 | ...
        download stream                               C block 0      | C block 1 | ...

    Per rank and call the host link carries (M / g + N / g) * K * 2 bytes up and N * M / g * 2 bytes down,
    against (M / g + N) * K * 2 up when every rank uploads all of B.  With one rank this is
    prism_b200.host.HostGemmBF16 (the library's host plan).  The reference's harness copies everything in,
    launches and copies everything out on one GPU (evals/h100_bench/main.cu:105-130).
    """

    def __init__(self, M: int, N: int, K: int, device, group: Any = None, steps: int = 0, gemm: Any = None,
                 overlap_download: bool | None = None, exchange: str | None = None, wait_limit_s: float = 0.0,
                 symmetric_bytes: Any = None):
        """`gemm(rows, n, K, A, B_block, C_block)` replaces the kernel call; the tests of the host-side
        logic pass a CPU stand-in together with device="cpu" (then there are no streams either).
        `overlap_download`: send blocks of C back while later blocks of B still go up (True, the default), or
        only after the last upload (False).  With several GPUs on one host, copies in both directions at once
        share the host's memory system (measured on a 4-GPU box: 55 GB/s up and 36-45 GB/s down per GPU when all
        copy one way, 38 and 23 when the directions mix), but the overlap still wins: 8192^3 on 4 GPUs 2.7 ms
        overlapped against 3.1 ms with the download held back."""
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device)
        self.on_cuda = self.device.type == "cuda"
        self.lo, self.hi = row_shard(M, self.world, self.rank)
        self.M, self.N, self.K = M, N, K
        self.rows = self.hi - self.lo
        self.single = None
        self._gemm = gemm
        self.overlap_download = True if overlap_download is None else bool(overlap_download)
        if self.world == 1 and gemm is None:
            from . import host
            self.single = host.HostGemmBF16(M, N, K, self.device)
            self.steps = self.single.blocks
            self.h2d_bytes, self.d2h_bytes = self.single.h2d_bytes, self.single.d2h_bytes
            return
        if steps == 0:
            steps = self._pick_steps(N, K)
        if steps < 1 or N % steps or (N // steps) % 128 or (N // steps) % self.world:
            raise ValueError(f"N={N} does not cut into {steps} blocks of a multiple of 128 rows that {self.world} ranks share")
        self.steps = steps
        self.block = N // steps                  # rows of B (columns of C) per step
        self.piece = self.block // self.world    # rows of B this rank uploads per step
        self.h2d_bytes = (self.rows + N // self.world) * K * 2
        self.d2h_bytes = N * self.rows * 2
        self.a = torch.empty((self.rows, K), dtype=torch.bfloat16, device=self.device)
        self.c = torch.empty((N, self.rows), dtype=torch.bfloat16, device=self.device)
        if exchange not in (None, "peer", "nccl"):
            raise ValueError("exchange must be 'peer' or 'nccl'")
        self.epoch = 0
        self.wait_limit_s = float(wait_limit_s)
        self.exchange = "nccl"
        if exchange != "nccl" and self.on_cuda and self.world > 1 and self.world <= 32:
            # two copies of B (by call parity) and steps * world flag words, in one peer-mapped allocation
            b_bytes = N * K * 2
            got = (symmetric_bytes or _symmetric_bytes)(2 * b_bytes + steps * self.world * 4, self.device, group)
            ok = torch.tensor([1 if got is not None else 0], dtype=torch.int32, device=self.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok.item()) == 1:
                raw, self._symm, bases = got
                self.b2 = raw[:2 * b_bytes].view(torch.bfloat16).view(2, N, K)
                self.flags = raw[2 * b_bytes:].view(torch.int32)
                self.flags.zero_()
                self._dst_table = torch.tensor(bases, dtype=torch.int64, device=self.device)
                self._flag_table = torch.tensor([p + 2 * b_bytes for p in bases], dtype=torch.int64, device=self.device)
                self._counter = torch.zeros(1, dtype=torch.int32, device=self.device)
                self.exchange = "peer"
                torch.cuda.synchronize(self.device)
                dist.barrier(group)   # every rank's flags are zero before anyone pushes
            elif exchange == "peer":
                raise RuntimeError("exchange='peer' needs peer-mapped (symmetric) memory on every rank")
        if self.exchange == "nccl":
            self.b2 = torch.empty((1, N, K), dtype=torch.bfloat16, device=self.device)
        # upload, gather, kernel, download
        self.lanes = [torch.cuda.Stream(self.device) for _ in range(4)] if self.on_cuda else [None] * 4

    def _pick_steps(self, N: int, K: int) -> int:
        """As many blocks as keep the kernels hidden behind the uploads: more blocks shorten what is left to do
        after the last byte has gone up (one block's gather, GEMM and download), but a block's GEMM takes a whole
        wave of the machine however few tiles it has, so the sum of the GEMMs must stay below the upload time.
        Rough machine constants (a B200 on PCIe 5): 55 GB/s up, 0.83 us per 64-wide k-block of a 512 x 256 tile,
        74 CTA pairs."""
        upload_ms = (self.rows + N // self.world) * K * 2 / 55e6
        wave_ms = (K / 64) * 0.83e-3
        for s in (16, 8, 4, 2, 1):
            if N % (s * 512) or (N // s) % (self.world * 8):
                continue
            tiles = max(1, self.rows // 256) * (N // s // 512)
            if s == 1 or s * wave_ms * -(-tiles // 74) <= 0.7 * upload_ms:
                return s
        return 0

    def __call__(self, A_host_local: torch.Tensor, B_host: torch.Tensor, C_host_local: torch.Tensor) -> torch.Tensor:
        if self.single is not None:
            return self.single(A_host_local, B_host, C_host_local)
        import contextlib
        for name, t, shape in (("A", A_host_local, (self.rows, self.K)), ("B", B_host, (self.N, self.K)),
                               ("C", C_host_local, (self.N, self.rows))):
            if t.device.type != "cpu" or t.dtype != torch.bfloat16 or tuple(t.shape) != shape or not t.is_contiguous():
                raise ValueError(f"{name} must be a contiguous host bf16 tensor of shape {shape}")
        import prism_b200 as pb
        from . import _lib
        gemm = self._gemm
        if gemm is None:
            gemm = pb.runmyh100
        up, gather, kernel, down = self.lanes
        cuda = self.on_cuda
        on = (lambda s: torch.cuda.stream(s)) if cuda else (lambda s: contextlib.nullcontext())
        event = (lambda: torch.cuda.Event()) if cuda else (lambda: None)
        record = (lambda e, s: e.record(s)) if cuda else (lambda e, s: None)
        wait = (lambda s, e: s.wait_event(e)) if cuda else (lambda s, e: None)
        caller = torch.cuda.current_stream(self.device) if cuda else None
        begin = event()
        record(begin, caller)
        for s in self.lanes:
            wait(s, begin)
        a_done = event()
        all_up = event()
        self.epoch += 1
        peer = self.exchange == "peer"
        b = self.b2[self.epoch & 1] if peer else self.b2[0]
        if peer:
            lib = pb.load()
            row_bytes = self.K * 2
            parity_off = (self.epoch & 1) * self.N * row_bytes
        for i in range(self.steps):
            lo = i * self.block
            mine = slice(lo + self.rank * self.piece, lo + (self.rank + 1) * self.piece)
            uploaded, gathered, computed = event(), event(), event()
            with on(up):
                b[mine].copy_(B_host[mine], non_blocking=True)
                record(uploaded, up)
                if i == 0:          # A goes up while the first block is being gathered
                    self.a.copy_(A_host_local, non_blocking=True)
                    record(a_done, up)
                if i == self.steps - 1:
                    record(all_up, up)
                    if not self.overlap_download:
                        wait(down, all_up)   # the download stream was idle until here: nothing of C has gone back yet
            with on(gather):
                wait(gather, uploaded)
                if peer:
                    # one-sided: push this rank's piece into every other rank's copy of the block, then flag it
                    stream = ctypes.c_void_p(gather.cuda_stream)
                    _lib.check(lib.prism_b200_peer_push(
                        b[mine].data_ptr(), self.piece * row_bytes, self._dst_table.data_ptr(),
                        parity_off + mine.start * row_bytes, self.world, self.rank, self._flag_table.data_ptr(),
                        i * self.world + self.rank, self.epoch, self._counter.data_ptr(), stream))
                else:
                    # On the GPU in place: this rank's piece already sits at its position in the block.
                    piece = b[mine] if cuda else b[mine].clone()
                    if self.world > 1:
                        dist.all_gather_into_tensor(b[lo:lo + self.block], piece, group=self.group)
                record(gathered, gather)
            with on(kernel):
                if peer:
                    # the block is complete when every rank's flag of this step carries this call's epoch
                    _lib.check(lib.prism_b200_peer_wait(self.flags.data_ptr(), i * self.world, self.world, self.epoch,
                                                        int(self.wait_limit_s * 1e9), ctypes.c_void_p(kernel.cuda_stream)))
                else:
                    wait(kernel, gathered)
                if i == 0:
                    wait(kernel, a_done)
                gemm(self.rows, self.block, self.K, self.a, b[lo:lo + self.block], self.c[lo:lo + self.block])
                record(computed, kernel)
            if self.overlap_download or i == self.steps - 1:
                first = i if self.overlap_download else 0
                with on(down):
                    wait(down, computed)
                    lo_d = first * self.block
                    C_host_local[lo_d:lo + self.block].copy_(self.c[lo_d:lo + self.block], non_blocking=True)
        for s in self.lanes:
            done = event()
            record(done, s)
            wait(caller, done)
        return C_host_local


class ShardedHostSgemm:
    """C = alpha * A @ B + beta * C for operands in HOST memory on g GPUs (one process each), rows of M sharded.

    The fp32 counterpart of ShardedHostGemmBF16.  Every rank holds its rows of A and C and all of B (K x N,
    the same on every rank) in pinned host memory.  Each rank uploads only rows [r * K / g, (r + 1) * K / g) of B
    and pushes them into every other rank's copy over NVLink (prism_b200_peer_push, one-sided, own kernel); its
    rows of A and C go up meanwhile, in blocks.  Every output element needs all of B, so the kernels start when
    all ranks' flags are up (prism_b200_peer_wait) and then run block by block of rows while later blocks of A and
    C still go up and finished blocks of C go back.  Per rank and call the host link carries
    (M / g * (K + N) + K / g * N) * 4 bytes up and M / g * N * 4 down, against (M / g * (K + N) + K * N) * 4 up when
    every rank uploads all of B.  With one rank, or without peer-mapped memory, it is
    prism_b200.host.HostSgemm on the rank's rows.  The reference's harness copies everything in, launches and
    copies everything out on one GPU (evals/4090_sgemm/main.cu:64-120)."""

    def __init__(self, M: int, N: int, K: int, device, group: Any = None, kernel: int = 5, block_rows: int = 0,
                 wait_limit_s: float = 0.0, symmetric_bytes: Any = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device)
        self.lo, self.hi = row_shard(M, self.world, self.rank)
        self.M, self.N, self.K, self.kernel = M, N, K, kernel
        self.rows = self.hi - self.lo
        self.wait_limit_s = float(wait_limit_s)
        self.epoch = 0
        self.single = None
        peer = self.world > 1 and self.world <= 32 and self.device.type == "cuda" and K % self.world == 0 and \
            (K // self.world * N * 4) % 16 == 0
        if peer:
            b_bytes = K * N * 4
            got = (symmetric_bytes or _symmetric_bytes)(2 * b_bytes + self.world * 4, self.device, group)
            ok = torch.tensor([1 if got is not None else 0], dtype=torch.int32, device=self.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            peer = int(ok.item()) == 1
        if not peer:
            from . import host
            self.single = host.HostSgemm(self.rows, N, K, self.device, kernel=kernel, block_rows=block_rows)
            self.h2d_bytes, self.d2h_bytes, self.blocks = self.single.h2d_bytes, self.single.d2h_bytes, self.single.blocks
            self.exchange = "none"
            return
        raw, self._symm, bases = got
        self.b2 = raw[:2 * b_bytes].view(torch.float32).view(2, K, N)
        self.flags = raw[2 * b_bytes:].view(torch.int32)
        self.flags.zero_()
        self._dst_table = torch.tensor(bases, dtype=torch.int64, device=self.device)
        self._flag_table = torch.tensor([p + 2 * b_bytes for p in bases], dtype=torch.int64, device=self.device)
        self._counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.exchange = "peer"
        self.piece = K // self.world                               # rows of B this rank uploads
        block_rows = block_rows or 512     # large enough for the 128 x 128 tile form, small enough to pipeline
        self.spans = [(lo, min(lo + block_rows, self.rows)) for lo in range(0, self.rows, block_rows)]
        self.blocks = len(self.spans)
        self.h2d_bytes = (self.rows * (K + N) + self.piece * N) * 4
        self.d2h_bytes = self.rows * N * 4
        self.a = torch.empty((self.rows, K), dtype=torch.float32, device=self.device)
        self.c = torch.empty((self.rows, N), dtype=torch.float32, device=self.device)
        self.lanes = [torch.cuda.Stream(self.device) for _ in range(4)]   # upload, exchange, kernel, download
        torch.cuda.synchronize(self.device)
        dist.barrier(group)   # every rank's flags are zero before anyone pushes

    def __call__(self, alpha: float, A_host_local: torch.Tensor, B_host: torch.Tensor, beta: float,
                 C_host_local: torch.Tensor) -> torch.Tensor:
        if self.single is not None:
            return self.single(alpha, A_host_local, B_host, beta, C_host_local)
        import prism_b200 as pb
        from . import _lib
        for name, t, shape in (("A", A_host_local, (self.rows, self.K)), ("B", B_host, (self.K, self.N)),
                               ("C", C_host_local, (self.rows, self.N))):
            if t.device.type != "cpu" or t.dtype != torch.float32 or tuple(t.shape) != shape or not t.is_contiguous():
                raise ValueError(f"{name} must be a contiguous host float32 tensor of shape {shape}")
        lib = pb.load()
        up, exchange, kernel, down = self.lanes
        caller = torch.cuda.current_stream(self.device)
        begin = torch.cuda.Event()
        begin.record(caller)
        for s in self.lanes:
            s.wait_event(begin)
        self.epoch += 1
        b = self.b2[self.epoch & 1]
        mine = slice(self.rank * self.piece, (self.rank + 1) * self.piece)
        row_bytes = self.N * 4
        b_up = torch.cuda.Event()
        with torch.cuda.stream(up):
            b[mine].copy_(B_host[mine], non_blocking=True)     # this rank's rows of B first: the others wait for them
            b_up.record(up)
        with torch.cuda.stream(exchange):
            exchange.wait_event(b_up)
            _lib.check(lib.prism_b200_peer_push(
                b[mine].data_ptr(), self.piece * row_bytes, self._dst_table.data_ptr(),
                (self.epoch & 1) * self.K * row_bytes + mine.start * row_bytes, self.world, self.rank,
                self._flag_table.data_ptr(), self.rank, self.epoch, self._counter.data_ptr(),
                ctypes.c_void_p(exchange.cuda_stream)))
        with torch.cuda.stream(kernel):
            _lib.check(lib.prism_b200_peer_wait(self.flags.data_ptr(), 0, self.world, self.epoch,
                                                int(self.wait_limit_s * 1e9), ctypes.c_void_p(kernel.cuda_stream)))
        for lo, hi in self.spans:
            uploaded, computed = torch.cuda.Event(), torch.cuda.Event()
            with torch.cuda.stream(up):
                self.a[lo:hi].copy_(A_host_local[lo:hi], non_blocking=True)
                self.c[lo:hi].copy_(C_host_local[lo:hi], non_blocking=True)
                uploaded.record(up)
            with torch.cuda.stream(kernel):
                kernel.wait_event(uploaded)
                pb.run_my_kernel(self.kernel, hi - lo, self.N, self.K, alpha, self.a[lo:hi], b, beta, self.c[lo:hi])
                computed.record(kernel)
            with torch.cuda.stream(down):
                down.wait_event(computed)
                C_host_local[lo:hi].copy_(self.c[lo:hi], non_blocking=True)
        for s in self.lanes:
            done = torch.cuda.Event()
            done.record(s)
            caller.wait_event(done)
        return C_host_local
