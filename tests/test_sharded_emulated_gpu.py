"""The peer-memory schedule of the sharded scan on ONE GPU: k "virtual ranks" whose word arrays all live
on the same device, with a device table of their k base addresses standing in for the peers' addresses.

Kernels of different ranks cannot wait for one another on one GPU (a launch that waits for a word that a
later launch stores would never see it), so each epoch first runs the reduce/publish step of every rank
and then the scan step of every rank -- the two-launch form of prism_b200_scan_sharded, and the older
three-piece form (reduce_u32, scan_publish_total, scan_seeded_peers).  Every word of the epoch is then in
place when a scan starts, and the concatenation of the chunks must equal the scan of the whole array bit
for bit, as the reference's harness checks element by element (evals/4090_scan/scan_harness.cuh:131-146).
The fused single launch (phases = 3) needs one GPU per rank and is covered by tests/test_sharded_gpu.py.
"""
import ctypes
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from oracle import cpu_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bounds(n, world):
    from prism_b200 import sharded
    return [sharded.chunk_bounds(n, world, r) for r in range(world)]


def _setup(world):
    """Per-rank word arrays (2 * world int64 each) in one allocation, and the device table of their addresses."""
    words = torch.zeros((world, 2 * world), dtype=torch.int64, device=DEV)
    table = torch.tensor([words[r].data_ptr() for r in range(world)], dtype=torch.int64, device=DEV)
    return words, table


@pytest.mark.parametrize("world,n,high", [(3, (1 << 22) + 12345, 1 << 20), (4, 3 * 4096 * 5 + 77, 0xFFFFFFFF),
                                          (4, 10, 16)])
@pytest.mark.parametrize("form", ["two_launch", "three_piece"])
def test_virtual_ranks_on_one_gpu(pb, world, n, high, form):
    lib = pb.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream(torch.device(DEV)).cuda_stream)
    words, table = _setup(world)
    spans = _bounds(n, world)           # n = 10 over 4 ranks: chunks of 4, 4, 2 and an empty one
    ws = [pb.scan_workspace(hi - lo, DEV) for lo, hi in spans]
    total = torch.zeros(1, dtype=torch.int32, device=DEV)
    with torch.cuda.device(DEV):
        for epoch in (1, 2, 3, 4):      # both halves of every word array, twice
            full = O.scan_inputs(n, seed=100 * world + epoch, high=high)
            expect = O.scan_cpu(full)
            chunks = [torch.from_numpy(full[lo:hi].view(np.int32).copy()).to(DEV) for lo, hi in spans]
            for r, x in enumerate(chunks):
                if form == "two_launch":
                    rc = lib.prism_b200_scan_sharded(x.numel(), x.data_ptr() if x.numel() else None, ws[r].data_ptr(),
                                                     words[r].data_ptr(), table.data_ptr(), r, world, epoch, 1, 0, stream)
                else:
                    rc = lib.prism_b200_reduce_u32(x.numel(), x.data_ptr() if x.numel() else None, total.data_ptr(), stream)
                    assert rc == 0, pb.last_error()
                    rc = lib.prism_b200_scan_publish_total(total.data_ptr(), table.data_ptr(), world, r, epoch, stream)
                assert rc == 0, pb.last_error()
            for r, x in enumerate(chunks):
                if form == "two_launch":
                    rc = lib.prism_b200_scan_sharded(x.numel(), x.data_ptr() if x.numel() else None, ws[r].data_ptr(),
                                                     words[r].data_ptr(), table.data_ptr(), r, world, epoch, 2, 0, stream)
                elif x.numel():
                    rc = lib.prism_b200_scan_seeded_peers(x.numel(), x.data_ptr(), ws[r].data_ptr(), words[r].data_ptr(),
                                                          r, world, epoch, stream)
                assert rc == 0, pb.last_error()
            torch.cuda.synchronize()
            assert pb.last_error()[0] == 0, pb.last_error()
            got = np.concatenate([x.cpu().numpy().view(np.uint32) for x in chunks])
            assert np.array_equal(got, expect), f"epoch {epoch}: first mismatch at {int(np.argmax(got != expect))}"
            # every rank's array holds every rank's {epoch, total} word of this epoch
            half = (epoch & 1) * world
            w = words[:, half:half + world].cpu().numpy().view(np.uint64)
            assert np.all((w & 0xFFFFFFFF) == epoch)
            totals = [int(full[lo:hi].sum(dtype=np.uint64)) & 0xFFFFFFFF for lo, hi in spans]
            assert np.all((w >> 32) == np.array(totals, dtype=np.uint64)[None, :])


@pytest.mark.parametrize("world,n", [(2, (1 << 22) + 4096), (3, 5 * 4096 * 7 + 8), (4, 200)])
def test_head_and_tail_on_virtual_rank_zero(pb, world, n):
    """The head_tail schedule with virtual ranks on one GPU: rank 0 scans the head outright and publishes its last
    element as its total, ranks 1 .. add up and publish their chunks, then every rank scans -- rank 0 its tail, as the
    piece behind all chunks (rank = world, scan phase only), which starts from the sum of all totals.  The pieces,
    put back in array order, equal the scan of the whole array bit for bit; three epochs."""
    from prism_b200 import sharded
    lib = pb.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream(torch.device(DEV)).cuda_stream)
    words, table = _setup(world)
    head, chunk, tail = sharded.head_tail_bounds(n, world)
    ws = [pb.scan_workspace(max(chunk, tail, head, 1), DEV) for _ in range(world + 1)]
    zero = torch.zeros(1, dtype=torch.int32, device=DEV)
    with torch.cuda.device(DEV):
        for epoch in (1, 2, 3):
            full = O.scan_inputs(n, seed=7 * world + epoch, high=1 << 24)
            expect = O.scan_cpu(full)
            parts = {r: [torch.from_numpy(full[a:b].view(np.int32).copy()).to(DEV) for a, b in
                         sharded.head_tail_pieces(n, world, r)] for r in range(world)}
            h, t = parts[0]
            if h.numel():
                assert lib.prism_b200_scan(h.numel(), h.data_ptr(), ws[world].data_ptr(), stream) == 0
            rc = lib.prism_b200_scan_publish_total((h[-1:] if h.numel() else zero).data_ptr(), table.data_ptr(), world, 0, epoch,
                                                   stream)
            assert rc == 0, pb.last_error()
            for r in range(1, world):
                x = parts[r][0]
                rc = lib.prism_b200_scan_sharded(x.numel(), x.data_ptr() if x.numel() else None, ws[r].data_ptr(),
                                                 words[r].data_ptr(), table.data_ptr(), r, world, epoch, 1, 0, stream)
                assert rc == 0, pb.last_error()
            rc = lib.prism_b200_scan_sharded(t.numel(), t.data_ptr() if t.numel() else None, ws[0].data_ptr(), words[0].data_ptr(),
                                             table.data_ptr(), world, world, epoch, 2, 0, stream)
            assert rc == 0, pb.last_error()
            for r in range(1, world):
                x = parts[r][0]
                rc = lib.prism_b200_scan_sharded(x.numel(), x.data_ptr() if x.numel() else None, ws[r].data_ptr(),
                                                 words[r].data_ptr(), table.data_ptr(), r, world, epoch, 2, 0, stream)
                assert rc == 0, pb.last_error()
            torch.cuda.synchronize()
            assert pb.last_error()[0] == 0, pb.last_error()
            got = np.concatenate([h.cpu().numpy()] + [parts[r][0].cpu().numpy() for r in range(1, world)] +
                                 [t.cpu().numpy()]).view(np.uint32)
            assert np.array_equal(got, expect), f"epoch {epoch}: first mismatch at {int(np.argmax(got != expect))}"
    # the piece behind all chunks exists for the scan phase only
    assert lib.prism_b200_scan_sharded(16, t.data_ptr(), ws[0].data_ptr(), words[0].data_ptr(), table.data_ptr(), world, world,
                                       4, 3, 0, stream) == 1
    pb.clear_error()


def test_scan_step_gives_up_when_a_word_never_arrives(pb):
    """Nothing publishes rank 1's word: the scan step of rank 0 must come back after its (short) limit with
    a device time-out recorded, and the context must stay usable."""
    lib = pb.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream(torch.device(DEV)).cuda_stream)
    world, n = 2, 3 * 4096 + 5
    words, table = _setup(world)
    x = torch.ones(n, dtype=torch.int32, device=DEV)
    ws = pb.scan_workspace(n, DEV)
    with torch.cuda.device(DEV):
        assert lib.prism_b200_scan_sharded(n, x.data_ptr(), ws.data_ptr(), words[0].data_ptr(), table.data_ptr(), 0, world,
                                           1, 1, 0, stream) == 0
        assert lib.prism_b200_scan_sharded(n, x.data_ptr(), ws.data_ptr(), words[0].data_ptr(), table.data_ptr(), 0, world,
                                           1, 2, 2_000_000, stream) == 0        # 2 ms for the peers
        torch.cuda.synchronize()
    code, msg = pb.last_error()
    assert code == 5 and "scan" in msg
    pb.clear_error()
    y = torch.ones(n, dtype=torch.int32, device=DEV)
    pb.scan_(y)
    torch.cuda.synchronize()
    assert int(y[-1]) == n and pb.last_error()[0] == 0


def test_one_sided_gather_with_virtual_ranks(pb):
    """prism_b200_peer_push / prism_b200_peer_wait with three virtual ranks whose buffers and flag arrays live on one
    device: every rank pushes its piece into the others' buffers, then every rank's wait finds all flags raised and
    every buffer holds the whole block.  Two epochs; a wait for an epoch nobody has pushed runs out and says so."""
    lib = pb.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream(torch.device(DEV)).cuda_stream)
    world, piece = 3, 1 << 20                     # bytes per rank and block
    bufs = torch.zeros((world, world * piece), dtype=torch.uint8, device=DEV)
    flags = torch.zeros((world, 8), dtype=torch.int32, device=DEV)
    dst_table = torch.tensor([bufs[r].data_ptr() for r in range(world)], dtype=torch.int64, device=DEV)
    flag_table = torch.tensor([flags[r].data_ptr() for r in range(world)], dtype=torch.int64, device=DEV)
    counter = torch.zeros(1, dtype=torch.int32, device=DEV)
    with torch.cuda.device(DEV):
        for epoch in (1, 2):
            g = torch.Generator(device=DEV).manual_seed(epoch)
            want = torch.randint(0, 256, (world * piece,), dtype=torch.uint8, device=DEV, generator=g)
            bufs.zero_()
            for r in range(world):                # a rank's own piece is in place before it pushes
                bufs[r, r * piece:(r + 1) * piece] = want[r * piece:(r + 1) * piece]
            for r in range(world):
                rc = lib.prism_b200_peer_push(bufs[r, r * piece:].data_ptr(), piece, dst_table.data_ptr(), r * piece, world, r,
                                              flag_table.data_ptr(), 2 + r, epoch, counter.data_ptr(), stream)
                assert rc == 0, pb.last_error()
            for r in range(world):
                assert lib.prism_b200_peer_wait(flags[r].data_ptr(), 2, world, epoch, 0, stream) == 0
            torch.cuda.synchronize()
            assert pb.last_error()[0] == 0, pb.last_error()
            assert all(torch.equal(bufs[r], want) for r in range(world))
            assert bool((flags[:, 2:2 + world] == epoch).all()) and int(counter[0]) == 0
        # an earlier epoch's wait is satisfied by a later flag; a later epoch's wait runs out (2 ms) and is reported
        assert lib.prism_b200_peer_wait(flags[0].data_ptr(), 2, world, 1, 0, stream) == 0
        torch.cuda.synchronize()
        assert pb.last_error()[0] == 0
        assert lib.prism_b200_peer_wait(flags[0].data_ptr(), 2, world, 3, 2_000_000, stream) == 0
        torch.cuda.synchronize()
    code, msg = pb.last_error()
    assert code == 5 and "peers" in msg
    pb.clear_error()
    assert lib.prism_b200_peer_push(bufs.data_ptr() + 8, 16, dst_table.data_ptr(), 0, world, 0, flag_table.data_ptr(), 0, 1,
                                    counter.data_ptr(), None) == 3     # misaligned source
    assert lib.prism_b200_peer_wait(flags.data_ptr(), 0, 33, 1, 0, None) == 1
    pb.clear_error()


def test_argument_checks(pb):
    lib = pb.load()
    words, table = _setup(2)
    x = torch.zeros(16, dtype=torch.int32, device=DEV)
    ws = pb.scan_workspace(16, DEV)
    args = (16, x.data_ptr(), ws.data_ptr(), words[0].data_ptr(), table.data_ptr())
    assert lib.prism_b200_scan_sharded(*args, 0, 2, 0, 3, 0, None) == 1      # epoch 0
    assert lib.prism_b200_scan_sharded(*args, 2, 2, 1, 3, 0, None) == 1      # rank outside the world
    assert lib.prism_b200_scan_sharded(*args, 0, 2, 1, 4, 0, None) == 1      # unknown phase bits
    assert lib.prism_b200_scan_sharded(*args, 0, 33, 1, 3, 0, None) == 1     # more than 32 ranks
    pb.clear_error()
