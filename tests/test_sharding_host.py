"""Host-side logic of the sharded paths, run as two gloo ranks on CPU.

The kernels are replaced by a stand-in that performs the same four operations
with the CPU oracle, so what is exercised here is the partitioning, the
all-gather of shard totals and the carry arithmetic -- not a product code path.
"""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from oracle import cpu_oracle as O  # noqa: E402
from prism_b200 import sharded  # noqa: E402


class OracleOps:
    """Same interface as the CUDA ops, computed with the oracle on CPU tensors."""

    def workspace(self, n, device):
        return torch.empty(0)

    @staticmethod
    def _np(t):
        return t.numpy().view(np.uint32)

    def reduce_u32(self, x, total):
        s = int(np.sum(self._np(x), dtype=np.uint64) & 0xFFFFFFFF)
        total[0] = s - (1 << 32) if s >= (1 << 31) else s  # the same 32 bits in an int32 tensor

    def _carry(self, totals, rank):
        return int(np.sum(self._np(totals)[:rank], dtype=np.uint64) & 0xFFFFFFFF)

    def scan_seeded_(self, x, workspace, totals, rank):
        v = self._np(x)
        v[:] = (O.scan_cpu(v).astype(np.uint64) + self._carry(totals, rank)).astype(np.uint32)

    def scan_(self, x, workspace):
        v = self._np(x)
        v[:] = O.scan_cpu(v)

    def scan_add_carry_(self, x, totals, rank):
        v = self._np(x)
        v[:] = (v.astype(np.uint64) + self._carry(totals, rank)).astype(np.uint32)

    def scan_sharded_(self, x, workspace, slots, peer_slots_dev, rank, world, epoch, wait_limit_s):
        """What the fused kernel does, with the peer stores replaced by an all-gather: every rank's
        {epoch, total} word lands in slot (epoch & 1) * world + r of this rank's array."""
        total = int(np.sum(self._np(x), dtype=np.uint64) & 0xFFFFFFFF)
        w = (total << 32) | epoch
        word = torch.tensor([w - (1 << 64) if w >= (1 << 63) else w], dtype=torch.int64)   # the same 64 bits
        words = torch.zeros(world, dtype=torch.int64)
        dist.all_gather_into_tensor(words, word)
        half = (epoch & 1) * world
        slots[half:half + world] = words
        assert all((int(w) & 0xFFFFFFFF) == epoch for w in words.tolist())
        carry = sum((int(w) >> 32) & 0xFFFFFFFF for w in words.tolist()[:rank]) & 0xFFFFFFFF
        v = self._np(x)
        v[:] = (O.scan_cpu(v).astype(np.uint64) + carry).astype(np.uint32)

    def scan_head_tail_(self, head, tail, ws_head, ws_tail, zero, slots, peer_slots_dev, world, epoch, wait_limit_s):
        """Rank 0 of the head_tail schedule: its word carries the head's total; the tail starts from all totals."""
        h = self._np(head)
        h[:] = O.scan_cpu(h)
        total = int(h[-1]) if h.size else 0
        w = (total << 32) | epoch
        word = torch.tensor([w - (1 << 64) if w >= (1 << 63) else w], dtype=torch.int64)
        words = torch.zeros(world, dtype=torch.int64)
        dist.all_gather_into_tensor(words, word)
        half = (epoch & 1) * world
        slots[half:half + world] = words
        carry = sum((int(w) >> 32) & 0xFFFFFFFF for w in words.tolist()) & 0xFFFFFFFF
        v = self._np(tail)
        v[:] = (O.scan_cpu(v).astype(np.uint64) + carry).astype(np.uint32)

    def check(self, device):
        pass


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _local_words(n_words, device, group):
    """Stand-in for symmetric memory on CPU: a private array (OracleOps fills it with an all-gather)."""
    return torch.zeros(n_words, dtype=torch.int64), None, 0


def _no_words(n_words, device, group):
    return None   # what _symmetric_words returns when there is no peer access


def _worker(rank, world, port, n, schedule, high, q, words="local"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = O.scan_inputs(n, seed=77, high=high)
        lo, hi = sharded.chunk_bounds(n, world, rank)
        scan = sharded.ShardedScan(hi - lo, "cpu", schedule=schedule, ops=OracleOps(),
                                   symmetric_words=_local_words if words == "local" else _no_words)
        expect = O.scan_cpu(full)[lo:hi]
        ok = True
        for _ in range(3):   # three epochs: both halves of the word array, and the first one again
            x = torch.from_numpy(full[lo:hi].copy().view(np.int32))
            scan(x)
            ok = ok and np.array_equal(x.numpy().view(np.uint32), expect)
        q.put((rank, ok, scan.totals_int64(), scan.schedule))
    finally:
        dist.destroy_process_group()


def _run_two_ranks(n, schedule, high, words="local"):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n, schedule, high, q, words)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return results


# n = 3 leaves the second rank with an empty chunk.
@pytest.mark.parametrize("schedule", sharded.ShardedScan.SCHEDULES + (sharded.ShardedScan.PEER_SCHEDULE,))
@pytest.mark.parametrize("n,high", [(100000, 16), (4099, 0xFFFFFFFF), (7, 2), (3, 9)])
def test_sharded_scan_two_ranks(schedule, n, high):
    results = _run_two_ranks(n, schedule, high)
    full = O.scan_inputs(n, seed=77, high=high)
    for rank, ok, totals, used in results:
        assert used == schedule
        assert ok, f"rank {rank} shard differs from the scan of the whole array"
        lo0, hi0 = sharded.chunk_bounds(n, 2, 0)
        assert totals[0] == int(full[lo0:hi0].sum(dtype=np.uint64)) & 0xFFFFFFFF


def test_peer_words_falls_back_when_there_is_no_symmetric_memory():
    """Without peer-writable words (no peer access, several nodes) every rank must end up on the same
    collective schedule and still produce the scan of the whole array."""
    for rank, ok, totals, used in _run_two_ranks(5000, sharded.ShardedScan.PEER_SCHEDULE, 16, words="none"):
        assert used == "reduce_then_scan"
        assert ok


def test_chunk_bounds_cover_and_align():
    for n in (0, 1, 5, 4096, 1 << 20, (1 << 20) + 3):
        for world in (1, 2, 3, 4, 8):
            spans = [sharded.chunk_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and a <= b
            for lo, _ in spans:
                assert lo % 4 == 0 or lo == n


def test_row_shard():
    assert sharded.row_shard(8192, 8, 3) == (3072, 4096)
    with pytest.raises(ValueError):
        sharded.row_shard(8192, 3, 0)
    with pytest.raises(ValueError):
        sharded.row_shard(1024, 16, 0)  # 64 rows per rank is not a multiple of the 128-row tile


def _gemm_worker(rank, world, port, q):
    """Host-side logic of the sharded host-buffer GEMM: which rows of B each rank uploads, the in-place
    gather of each block and the block-wise GEMM, with the kernel replaced by a float64 product on the CPU."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, N, K = 256 * world, 1024, 64
        A, B = O.gemm_bf16_inputs(M, N, K, seed=12)
        a_all = torch.from_numpy(A.view(np.int16)).view(torch.bfloat16)
        b_all = torch.from_numpy(B.view(np.int16)).view(torch.bfloat16)

        def gemm(rows, n, k, a, b_block, c_block):
            c_block.copy_((b_block.double() @ a.double().t()).to(torch.bfloat16))

        op = sharded.ShardedHostGemmBF16(M, N, K, "cpu", gemm=gemm, steps=2)
        assert op.steps == 2 and op.block == 512 and op.piece == 512 // world
        # a rank only ever reads its own pieces of B: everything else is poisoned in its host copy
        b_host = torch.full_like(b_all, float("nan"))
        for i in range(op.steps):
            mine = slice(i * op.block + rank * op.piece, i * op.block + (rank + 1) * op.piece)
            b_host[mine] = b_all[mine]
        c_host = torch.empty((N, op.rows), dtype=torch.bfloat16)
        op(a_all[op.lo:op.hi].contiguous(), b_host, c_host)
        ref = O.gemm_bf16_cpu(A[op.lo:op.hi], B)
        ok, worst = O.gemm_bf16_check(c_host.view(torch.int16).numpy().view(np.uint16), ref)
        # the same with C sent back in one piece after the last upload
        late = sharded.ShardedHostGemmBF16(M, N, K, "cpu", gemm=gemm, steps=2, overlap_download=False)
        c_late = torch.full((N, op.rows), float("nan"), dtype=torch.bfloat16)
        late(a_all[op.lo:op.hi].contiguous(), b_host, c_late)
        ok = ok and torch.equal(c_late, c_host)
        q.put((rank, ok, worst, op.h2d_bytes, op.d2h_bytes))
    finally:
        dist.destroy_process_group()


def test_sharded_host_gemm_uploads_each_row_of_b_once_across_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gemm_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, worst, h2d, d2h in results:
        assert ok, (rank, worst)
        assert h2d == (256 + 512) * 64 * 2 and d2h == 1024 * 256 * 2


def _head_tail_worker(rank, world, port, n, high, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = O.scan_inputs(n, seed=91, high=high)
        pieces = sharded.head_tail_pieces(n, world, rank)
        local = np.concatenate([full[lo:hi] for lo, hi in pieces])
        expect = np.concatenate([O.scan_cpu(full)[lo:hi] for lo, hi in pieces])
        head = pieces[0][1] - pieces[0][0] if rank == 0 else 0
        scan = sharded.ShardedScan(local.size, "cpu", schedule="head_tail", ops=OracleOps(), symmetric_words=_local_words,
                                   head=head)
        ok = True
        for _ in range(3):
            x = torch.from_numpy(local.copy().view(np.int32))
            scan(x)
            ok = ok and np.array_equal(x.numpy().view(np.uint32), expect)
        q.put((rank, ok, scan.schedule, pieces))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n,high", [(2, 100000, 16), (2, 4099, 0xFFFFFFFF), (2, 40, 3), (3, 70001, 1 << 20)])
def test_head_tail_schedule(world, n, high):
    """Rank 0 owns the head and the tail of the array and never adds its pieces up first; the other ranks the chunks
    between them.  The pieces cover the array, and every piece equals the scan of the whole array on its range."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_head_tail_worker, args=(r, world, port, n, high, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    covered = sorted(rng for _, _, _, pieces in results for rng in pieces)
    assert covered[0][0] == 0 and covered[-1][1] == n and all(a[1] == b[0] for a, b in zip(covered, covered[1:]))
    for rank, ok, used, _ in results:
        assert used == "head_tail" and ok, f"rank {rank}"


def test_head_tail_bounds():
    for n, world in [(1 << 30, 2), (1 << 30, 8), (100000, 3), (40, 2), (17, 4)]:
        b = sharded.head_tail_bounds(n, world)
        if b is None:
            continue
        head, chunk, tail = b
        assert head == chunk // 2 and 0 <= tail <= chunk and head + (world - 1) * chunk + tail == n
        assert head % 4 == 0 and chunk % 8 == 0
    head, chunk, tail = sharded.head_tail_bounds(1 << 30, 2)
    assert abs(chunk - (1 << 30) / 2.5) < 32 and abs(tail - chunk) < 32        # rank 0 owns 1.5 chunks, 8 B/element
    assert sharded.head_tail_bounds(100, 1) is None and sharded.head_tail_bounds(3, 8) is None
