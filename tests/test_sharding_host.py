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


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, schedule, high, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = O.scan_inputs(n, seed=77, high=high)
        lo, hi = sharded.chunk_bounds(n, world, rank)
        x = torch.from_numpy(full[lo:hi].copy().view(np.int32))
        scan = sharded.ShardedScan(hi - lo, "cpu", schedule=schedule, ops=OracleOps())
        scan(x)
        expect = O.scan_cpu(full)[lo:hi]
        ok = np.array_equal(x.numpy().view(np.uint32), expect)
        q.put((rank, ok, scan.totals_int64()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("schedule", sharded.ShardedScan.SCHEDULES)
@pytest.mark.parametrize("n,high", [(100000, 16), (4099, 0xFFFFFFFF), (7, 2)])
def test_sharded_scan_two_ranks(schedule, n, high):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n, schedule, high, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    full = O.scan_inputs(n, seed=77, high=high)
    for rank, ok, totals in results:
        assert ok, f"rank {rank} shard differs from the scan of the whole array"
        lo0, hi0 = sharded.chunk_bounds(n, 2, 0)
        assert totals[0] == int(full[lo0:hi0].sum(dtype=np.uint64)) & 0xFFFFFFFF


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
