"""Host-buffer operators (prism_b200.host over the library's host plans): pinned host tensors in, pinned host tensors
out, blocks pipelined over three streams.  Results must equal the device-resident entry points bit for bit (same kernels, same k order), and
the oracle."""
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


@pytest.fixture(scope="module")
def pb():
    import prism_b200
    prism_b200.load()
    return prism_b200


@pytest.mark.parametrize("n,block", [(1 << 20, 1 << 18), (3 * (1 << 20) + 8, 1 << 20), (1000, None), (4, None)])
def test_host_scan_blocks_chain(pb, n, block):
    from prism_b200 import host
    x = O.scan_inputs(n, seed=n)
    xh = torch.from_numpy(x.view(np.int32).copy()).pin_memory()
    op = host.HostScan(n, DEV, block_elems=block or 0)
    if block is not None and n > block:
        assert op.blocks > 1
    for _ in range(2):      # twice: the carry is re-armed per call
        xh.copy_(torch.from_numpy(x.view(np.int32)))
        op(xh)
        torch.cuda.synchronize()
        assert np.array_equal(xh.numpy().view(np.uint32), O.scan_cpu(x))


def test_host_gemm_bf16_blocks(pb):
    from prism_b200 import host
    M, N, K = 512, 2048, 256
    A, B = O.gemm_bf16_inputs(M, N, K, seed=5)
    a = torch.from_numpy(A.view(np.int16)).view(torch.bfloat16)
    b = torch.from_numpy(B.view(np.int16)).view(torch.bfloat16)
    ah, bh = a.pin_memory(), b.pin_memory()
    ch = torch.empty((N, M), dtype=torch.bfloat16).pin_memory()
    op = host.HostGemmBF16(M, N, K, DEV, block_rows=512)
    assert op.blocks == 4
    op(ah, bh, ch)
    torch.cuda.synchronize()
    c = torch.empty((N, M), dtype=torch.bfloat16, device=DEV)
    pb.runmyh100(M, N, K, a.to(DEV), b.to(DEV), c)
    torch.cuda.synchronize()
    got = ch.float().numpy()
    ref = O.gemm_bf16_cpu(A, B)          # (N, M) fp64 of the bf16-rounded inputs
    rms = float(np.sqrt(np.mean(ref * ref)))
    assert np.all(np.abs(got - ref) <= 1e-2 * np.abs(ref) + 1e-2 * rms)
    # the whole-matrix call may pick another tile form, but every form accumulates k in the same order
    assert torch.equal(ch, c.cpu())


def test_host_sgemm_blocks(pb):
    from prism_b200 import host
    M, N, K = 1024, 384, 256
    A, B, C = O.sgemm_inputs(M, N, K, seed=9)
    ah, bh, ch = (torch.from_numpy(t.copy()).pin_memory() for t in (A, B, C))
    op = host.HostSgemm(M, N, K, DEV, block_rows=256)
    assert op.blocks == 4
    op(1.5, ah, bh, 0.5, ch)
    torch.cuda.synchronize()
    assert O.sgemm_rel_error(ch.numpy(), O.sgemm_cpu(1.5, A, B, 0.5, C)) <= O.SGEMM_TOL
    # With no tile shared along K every tile form adds one element's products in the same order, so the plan's
    # blocks of rows and a whole-matrix call give the same bits whichever tiles they pick.
    lib = pb.load()
    try:
        assert lib.prism_b200_sgemm_k_slices(1) == 0
        ch.copy_(torch.from_numpy(C))
        op(1.5, ah, bh, 0.5, ch)
        c = torch.from_numpy(C).to(DEV)
        pb.run_my_kernel(5, M, N, K, 1.5, torch.from_numpy(A).to(DEV), torch.from_numpy(B).to(DEV), 0.5, c)
        torch.cuda.synchronize()
    finally:
        lib.prism_b200_sgemm_k_slices(-1)
    assert torch.equal(ch, c.cpu())
