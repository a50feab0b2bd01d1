"""The sharded paths on real GPUs: one child process per GPU over NCCL.  Needs at least two GPUs;
the host-side logic alone is covered on CPU by tests/test_sharding_host.py."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu

_RANK = r"""
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, %(root)r)
import prism_b200 as pb
from prism_b200 import sharded
from oracle import cpu_oracle as O

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
dev = torch.device("cuda", rank)

# scan: contiguous chunks of one seeded array, both schedules, ragged length
n = (1 << 22) + 12345
full = O.scan_inputs(n, seed=5, high=1 << 20)
expect = O.scan_cpu(full)
lo, hi = sharded.chunk_bounds(n, world, rank)
for schedule in (sharded.ShardedScan.PEER_SCHEDULE,) + sharded.ShardedScan.SCHEDULES:
    scan = sharded.ShardedScan(hi - lo, dev, schedule=schedule)
    for rep in range(3):   # repeated calls: epochs alternate between the two halves of the slot array
        x = torch.from_numpy(full[lo:hi].view(np.int32).copy()).to(dev)
        scan(x)
        torch.cuda.synchronize()
        assert np.array_equal(x.cpu().numpy().view(np.uint32), expect[lo:hi]), (schedule, rank, rep)
        assert sum(scan.totals_int64()) & 0xFFFFFFFF == int(expect[-1]), (schedule, rank, rep)
assert sharded.ShardedScan(hi - lo, dev).schedule == "peer_words"

# the fused launch with a longer limit and the checked mode; an array so short that the last rank's chunk is empty
for n_small in (3 * world + 1, 4 * (world - 1)):
    full_s = O.scan_inputs(n_small, seed=6, high=9)
    lo_s, hi_s = sharded.chunk_bounds(n_small, world, rank)
    scan = sharded.ShardedScan(hi_s - lo_s, dev, schedule="peer_words", wait_limit_s=5.0, checked=True)
    for rep in range(3):
        x = torch.from_numpy(full_s[lo_s:hi_s].view(np.int32).copy()).to(dev)
        scan(x)
        assert np.array_equal(x.cpu().numpy().view(np.uint32), O.scan_cpu(full_s)[lo_s:hi_s]), (n_small, rank, rep)

# the head_tail schedule: rank 0 owns the head and the tail of the array and never adds them up first
for n_ht in ((1 << 22) + 12345, 40 * world):
    full_h = O.scan_inputs(n_ht, seed=8, high=1 << 20)
    expect_h = O.scan_cpu(full_h)
    pieces = sharded.head_tail_pieces(n_ht, world, rank)
    local = np.concatenate([full_h[a:b] for a, b in pieces])
    want = np.concatenate([expect_h[a:b] for a, b in pieces])
    scan = sharded.ShardedScan(local.size, dev, schedule="head_tail", head=pieces[0][1] - pieces[0][0] if rank == 0 else 0,
                               wait_limit_s=5.0, checked=True)
    assert scan.schedule == "head_tail"
    for rep in range(4):
        x = torch.from_numpy(local.view(np.int32).copy()).to(dev)
        scan(x)
        torch.cuda.synchronize()
        assert np.array_equal(x.cpu().numpy().view(np.uint32), want), ("head_tail", n_ht, rank, rep)

# bf16 GEMM from host arrays: every rank uploads its rows of A and 1/world of B, B is completed over NVLink
Mh, Nh, Kh = 256 * world, 2048, 512
A, B = O.gemm_bf16_inputs(Mh, Nh, Kh, seed=19)
from prism_b200 import host
ref_c = None
for exchange in ("peer", "nccl"):   # one-sided pushes over peer memory (own kernels), and NCCL all-gathers
    op = sharded.ShardedHostGemmBF16(Mh, Nh, Kh, dev, steps=4, exchange=exchange)
    assert op.exchange == exchange
    if ref_c is None:
        ah = host.pinned_near(dev, (op.rows, Kh), torch.bfloat16); ah.copy_(torch.from_numpy(A[op.lo:op.hi].view(np.int16)).view(torch.bfloat16))
        bh = host.pinned_near(dev, (Nh, Kh), torch.bfloat16); bh.copy_(torch.from_numpy(B.view(np.int16)).view(torch.bfloat16))
        ch = host.pinned_near(dev, (Nh, op.rows), torch.bfloat16)
        ref_c = O.gemm_bf16_cpu(A[op.lo:op.hi], B)
    for rep in range(4):            # four calls: both copies of B, twice, and back-to-back without a host wait first
        ch.fill_(float("nan"))
        if (rep + rank) & 1:        # ranks enter the call tens of milliseconds apart, in changing order
            import time
            time.sleep(0.03)
        op(ah, bh, ch)
        if rep & 1:
            op(ah, bh, ch)
        torch.cuda.synchronize()
        ok, worst = O.gemm_bf16_check(ch.view(torch.int16).numpy().view(np.uint16), ref_c)
        assert ok, (exchange, rank, rep, worst)
    assert op.steps == 4 and op.h2d_bytes == (op.rows + Nh // world) * Kh * 2
    assert pb.last_error()[0] == 0, pb.last_error()

# bf16 GEMM: rows of M sharded, B replicated, no collective
M, N, K = 256 * world, 512, 256
A, B = O.gemm_bf16_inputs(M, N, K, seed=9)
plan = sharded.RowShardedGemmBF16(M, N, K)
a = torch.from_numpy(A[plan.lo:plan.hi].view(np.int16)).to(dev).view(torch.bfloat16)
b = torch.from_numpy(B.view(np.int16)).to(dev).view(torch.bfloat16)
c = torch.empty((N, plan.rows), dtype=torch.bfloat16, device=dev)
plan(a, b, c)
torch.cuda.synchronize()
ref = O.gemm_bf16_cpu(A[plan.lo:plan.hi], B)
ok, worst = O.gemm_bf16_check(c.view(torch.int16).cpu().numpy().view(np.uint16), ref)
assert ok, worst

# SGEMM the same way
A, B, C = O.sgemm_inputs(M, 256, 128, seed=3)
sp = sharded.RowShardedSgemm(M, 256, 128)
ta, tb, tc = (torch.from_numpy(np.ascontiguousarray(t)).to(dev) for t in (A[sp.lo:sp.hi], B, C[sp.lo:sp.hi]))
sp(1.5, ta, tb, 0.5, tc)
torch.cuda.synchronize()
err = O.sgemm_rel_error(tc.cpu().numpy(), O.sgemm_cpu(1.5, A[sp.lo:sp.hi], B, 0.5, C[sp.lo:sp.hi]))
assert err <= O.SGEMM_TOL, err
# SGEMM from host arrays: every rank uploads 1 / world of B's rows and pushes them to the others
Ms, Ns, Ks = 256 * world, 384, 128 * world
A, B, C = O.sgemm_inputs(Ms, Ns, Ks, seed=23)
hs = sharded.ShardedHostSgemm(Ms, Ns, Ks, dev, block_rows=128)
assert hs.exchange == "peer" and hs.blocks == 2 and hs.h2d_bytes == (hs.rows * (Ks + Ns) + Ks // world * Ns) * 4
ha, hb = (torch.from_numpy(np.ascontiguousarray(t)).pin_memory() for t in (A[hs.lo:hs.hi], B))
want = O.sgemm_cpu(1.5, A[hs.lo:hs.hi], B, 0.5, C[hs.lo:hs.hi])
for rep in range(3):
    hc = torch.from_numpy(np.ascontiguousarray(C[hs.lo:hs.hi])).pin_memory()
    hs(1.5, ha, hb, 0.5, hc)
    torch.cuda.synchronize()
    err = O.sgemm_rel_error(hc.numpy(), want)
    assert err <= O.SGEMM_TOL, (rank, rep, err)
assert pb.last_error()[0] == 0, pb.last_error()
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
"""


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_sharded_scan_and_gemm_over_nccl():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    port = _free_port()
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, "-c", _RANK % {"root": str(ROOT)}], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=600)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {rank} failed:\n{out[-3000:]}"
