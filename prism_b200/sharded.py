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

    def check(self, device):
        """Synchronise and raise if a device-side wait ran out."""
        import torch as _t
        _t.cuda.synchronize(device)
        code, msg = self._pb.last_error()
        if code:
            self._pb.clear_error()
            raise self._pb.PrismB200Error(code, msg)


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

    def __init__(self, n_local: int, device, group: Any = None, schedule: str | None = None, ops: Any = None,
                 wait_limit_s: float = 0.0, checked: bool = False, symmetric_words: Any = _symmetric_words):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        on_cuda = torch.device(device).type == "cuda"
        asked = schedule
        if schedule is None:
            schedule = self.PEER_SCHEDULE if (on_cuda and self.world > 1 and ops is None) else "reduce_then_scan"
        if schedule not in self.SCHEDULES + (self.PEER_SCHEDULE,):
            raise ValueError(f"schedule must be one of {self.SCHEDULES + (self.PEER_SCHEDULE,)}")
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
        self.workspace = self.ops.workspace(n_local, device)
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
            else:
                schedule = "reduce_then_scan"
        self.schedule = schedule
        self.fell_back = asked in (None, self.PEER_SCHEDULE) and schedule != self.PEER_SCHEDULE and on_cuda and self.world > 1

    def _exchange(self, total: torch.Tensor) -> None:
        if self.world == 1:
            self.totals.copy_(total)
        else:
            dist.all_gather_into_tensor(self.totals, total, group=self.group)

    def __call__(self, x_local: torch.Tensor) -> torch.Tensor:
        if x_local.numel() != self.n_local:
            raise ValueError(f"shard has {x_local.numel()} elements, planned for {self.n_local}")
        if self.schedule == self.PEER_SCHEDULE and self.world > 1:
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
