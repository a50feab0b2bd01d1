"""GPU parity of the scan: C ABI vs the CPU oracle, the golden fixture and the
reference's own scan_kernel recompiled for sm_100.  Bit-exact everywhere."""
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


def _run(pb, x_np):
    x = torch.from_numpy(x_np.view(np.int32).copy()).to(DEV)
    ws = pb.scan_workspace(x.numel(), DEV)
    ws.fill_(0xAB)  # the workspace may hold anything on entry
    pb.launch_scan(x.numel(), x, ws)
    torch.cuda.synchronize()
    return x.cpu().numpy().view(np.uint32)


# Sizes: empty, below one vector, ragged, the reference's correctness sizes
# (evals/4090_scan/main.cu:97-103: 16384, 32768, 2^20, 2^24, 2^26) and config #2 (2^24, values < 16).
@pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 127, 128, 4095, 4096, 4097, 8191, 16384, 32768, 100003,
                               1 << 20, (1 << 20) + 1, 1 << 24])
def test_scan_matches_oracle(pb, n):
    x = O.scan_inputs(n, seed=1000 + n % 97, high=16)
    assert np.array_equal(_run(pb, x), O.scan_cpu(x))


def test_scan_reference_harness_values(pb):
    x = O.scan_inputs(1 << 22, seed=0xCA7CAFE, high=101)  # uniform 0..100, scan_harness.cuh:172
    assert np.array_equal(_run(pb, x), O.scan_cpu(x))


def test_scan_wraparound(pb):
    x = O.scan_inputs((1 << 18) + 77, seed=5, high=0xFFFFFFFF)
    assert np.array_equal(_run(pb, x), O.scan_cpu(x))


def test_scan_golden_fixture(pb):
    g = np.load(ROOT / "tests" / "golden" / "scan_ref_cpu.npz")
    for key in ("small", "tile", "ragged", "wrap"):
        assert np.array_equal(_run(pb, g[key + "_in"]), g[key + "_out"]), key


def test_scan_uint32_dtype_and_workspace_reuse(pb):
    n = (1 << 16) + 9
    ws = pb.scan_workspace(n, DEV)
    for seed in range(3):  # same workspace, back to back, no host re-arming
        x_np = O.scan_inputs(n, seed=seed, high=1 << 20)
        x = torch.from_numpy(x_np.view(np.int32).copy()).to(DEV).view(torch.uint32)
        pb.launch_scan(n, x, ws)
        assert np.array_equal(x.view(torch.int32).cpu().numpy().view(np.uint32), O.scan_cpu(x_np))


def test_scan_2_26_largest_reference_correctness_size(pb):
    n = 1 << 26
    g = torch.Generator(device=DEV).manual_seed(26)
    x = torch.randint(0, 101, (n,), dtype=torch.int32, device=DEV, generator=g)
    x_np = x.cpu().numpy().view(np.uint32)
    pb.scan_(x)
    assert np.array_equal(x.cpu().numpy().view(np.uint32), O.scan_cpu(x_np))


def test_scan_2_28_properties(pb):
    """Benchmark size: values in {0,1}; checked by properties that need no CPU pass over
    the array: last element = int64 total, differences reproduce the input, monotone."""
    n = 1 << 28
    g = torch.Generator(device=DEV).manual_seed(28)
    x = torch.randint(0, 2, (n,), dtype=torch.int32, device=DEV, generator=g)
    inp = x.clone()
    total = int(inp.sum(dtype=torch.int64))
    pb.scan_(x)
    assert int(x[-1]) == total
    assert int(x[0]) == int(inp[0])
    assert torch.equal(x[1:] - x[:-1], inp[1:])
    # and against a sample of oracle values: the prefix at a few tile boundaries
    xs = x[: 1 << 22].cpu().numpy().view(np.uint32)
    assert np.array_equal(xs, O.scan_cpu(inp[: 1 << 22].cpu().numpy().view(np.uint32)))


def test_scan_2_30_properties(pb):
    """The sharded benchmark's total size on one GPU (4 GiB): last element = int64 total, differences
    reproduce the input, and the first and last 2^22 elements equal the oracle continued from the
    int64 prefix before them."""
    n = 1 << 30
    g = torch.Generator(device=DEV).manual_seed(30)
    x = torch.randint(0, 2, (n,), dtype=torch.int32, device=DEV, generator=g)
    head = x[: 1 << 22].cpu().numpy().view(np.uint32).copy()
    tail = x[-(1 << 22):].cpu().numpy().view(np.uint32).copy()
    total = int(x.sum(dtype=torch.int64))
    before_tail = int(x[: n - (1 << 22)].sum(dtype=torch.int64))
    first = int(x[0])
    # differences are checked in chunks against the input, which is regenerated from the same seed
    pb.scan_(x)
    assert int(x[-1]) == total and int(x[0]) == first
    g2 = torch.Generator(device=DEV).manual_seed(30)
    inp = torch.randint(0, 2, (n,), dtype=torch.int32, device=DEV, generator=g2)
    step = 1 << 28
    for lo in range(0, n, step):
        hi = min(n, lo + step)
        a = max(lo, 1)
        assert torch.equal(x[a:hi] - x[a - 1:hi - 1], inp[a:hi]), lo
    assert np.array_equal(x[: 1 << 22].cpu().numpy().view(np.uint32), O.scan_cpu(head))
    expect_tail = (O.scan_cpu(tail).astype(np.uint64) + before_tail).astype(np.uint32)
    assert np.array_equal(x[-(1 << 22):].cpu().numpy().view(np.uint32), expect_tail)


@pytest.mark.parametrize("n", [16384, 32768, 1 << 20, 1 << 24])
def test_scan_matches_reference_kernel(pb, ref_gpu, n):
    """Side by side with the reference's generated scan_kernel (recompiled for sm_100)."""
    x_np = O.scan_inputs(n, seed=n & 0xFFFF, high=16)
    mine = _run(pb, x_np)
    xr = torch.from_numpy(x_np.view(np.int32).copy()).to(DEV)
    ws = torch.empty(ref_gpu.ref_scan_workspace_size(n), dtype=torch.uint8, device=DEV)
    torch.cuda.synchronize()
    assert ref_gpu.ref_scan(n, xr.data_ptr(), ws.data_ptr()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(mine, xr.cpu().numpy().view(np.uint32))


def test_sharded_pieces_compose(pb):
    """reduce + seeded scan, and scan + carry add, over 3 uneven chunks on one GPU equal the full scan."""
    full = O.scan_inputs(300007, seed=8, high=1 << 30)
    cuts = [0, 100000, 100000, 233336, 300007]  # includes an empty chunk
    expect = O.scan_cpu(full)
    totals = torch.zeros(len(cuts) - 1, dtype=torch.int32, device=DEV)
    chunks = []
    for r in range(len(cuts) - 1):
        c = torch.from_numpy(full[cuts[r]:cuts[r + 1]].view(np.int32).copy()).to(DEV)
        pb.reduce_u32(c, totals[r:r + 1])
        chunks.append(c)
    torch.cuda.synchronize()
    tot_np = totals.cpu().numpy().view(np.uint32)
    for r in range(len(cuts) - 1):
        assert int(tot_np[r]) == int(full[cuts[r]:cuts[r + 1]].sum(dtype=np.uint64)) & 0xFFFFFFFF
    for r, c in enumerate(chunks):
        a = c.clone()
        pb.scan_seeded_(a, pb.scan_workspace(a.numel(), DEV), totals, r)
        b = c.clone()
        pb.scan_(b)
        pb.scan_add_carry_(b, totals, r)
        assert np.array_equal(a.cpu().numpy().view(np.uint32), expect[cuts[r]:cuts[r + 1]]), r
        assert np.array_equal(b.cpu().numpy().view(np.uint32), expect[cuts[r]:cuts[r + 1]]), r


@pytest.mark.parametrize("n", [1, 5, 4096, 4097, 100003, 1 << 22])
def test_scan_f32_exact_on_small_integers(pb, n):
    """fp32 flavour on integer-valued data whose partial sums all stay below 2^24: every fp32 add is exact,
    whatever the grouping, so the result must equal the running sum bit for bit."""
    rng = np.random.default_rng(n)
    x = rng.integers(0, 4, n).astype(np.float32)
    t = torch.from_numpy(x.copy()).to(DEV)
    pb.scan_f32_(t)
    torch.cuda.synchronize()
    assert np.array_equal(t.cpu().numpy().astype(np.float64), O.scan_f32_cpu(x))


@pytest.mark.parametrize("n,signed", [(1000003, False), (1 << 20, True), (1 << 24, False)])
def test_scan_f32_against_fp64(pb, n, signed):
    """Random data against the fp64 running sum.  An output is reached through at most 24 fp32 adds inside its
    tile (3 in a thread, 5 shuffle steps, 4 + 8 hand-offs, 2 offsets, the prefix) plus at most 2 per preceding tile
    along the chain of look-backs (when every look-back finds its prefix one tile back); each add rounds by at
    most 2^-24 of the running sum of |x|.  That worst case is the bound; typical errors are far below it."""
    rng = np.random.default_rng(n + signed)
    x = (rng.uniform(-1.0, 1.0, n) if signed else rng.uniform(0.0, 1.0, n)).astype(np.float32)
    t = torch.from_numpy(x.copy()).to(DEV)
    pb.scan_f32_(t)
    torch.cuda.synchronize()
    ref = O.scan_f32_cpu(x)
    scale = np.cumsum(np.abs(x).astype(np.float64))
    err = np.abs(t.cpu().numpy().astype(np.float64) - ref) / np.maximum(scale, 1.0)
    tiles = -(-n // 4096)
    assert err.max() <= (24 + 2 * tiles) * 2.0 ** -24, err.max()


@pytest.mark.parametrize("n", [1, 4, 4097, 100003, 1 << 22])
@pytest.mark.parametrize("exclusive", [False, True])
def test_scan_general_out_of_place_and_exclusive(pb, n, exclusive):
    """Separate output and the exclusive form, uint32: bit-exact against the oracle (exclusive = inclusive shifted
    by one element with a leading zero); the input is left untouched; in == out works as well."""
    x = O.scan_inputs(n, seed=n + exclusive, high=1 << 30)
    inc = O.scan_cpu(x)
    want = np.concatenate([np.zeros(1, np.uint32), inc[:-1]]) if exclusive else inc
    t = torch.from_numpy(x.view(np.int32).copy()).to(DEV)
    out = pb.scan(t, exclusive=exclusive)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want)
    assert np.array_equal(t.cpu().numpy().view(np.uint32), x)
    pb.scan(t, out=t, exclusive=exclusive)
    torch.cuda.synchronize()
    assert np.array_equal(t.cpu().numpy().view(np.uint32), want)


def test_scan_general_f32_exclusive(pb):
    n = 300007
    x = np.random.default_rng(3).integers(0, 4, n).astype(np.float32)     # exact in fp32
    out = pb.scan(torch.from_numpy(x).to(DEV), exclusive=True)
    torch.cuda.synchronize()
    want = np.concatenate([[0.0], O.scan_f32_cpu(x)[:-1]])
    assert np.array_equal(out.cpu().numpy().astype(np.float64), want)


@pytest.mark.parametrize("n", [1, 2, 3, 2047, 2048, 2049, 100003, (1 << 22) + 1])
@pytest.mark.parametrize("exclusive", [False, True])
def test_scan_int64(pb, n, exclusive):
    """64-bit integer flavour (2048-element tiles, a record in two words): full-range values, so that sums wrap
    around 2^64 and both halves of every record matter; bit-exact against the oracle, out of place and in place."""
    rng = np.random.default_rng(n * 2 + exclusive)
    x = rng.integers(0, 1 << 64, n, dtype=np.uint64)
    inc = O.scan_i64_cpu(x)
    want = np.concatenate([np.zeros(1, np.uint64), inc[:-1]]) if exclusive else inc
    t = torch.from_numpy(x.view(np.int64).copy()).to(DEV)
    out = pb.scan(t, exclusive=exclusive)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint64), want)
    assert np.array_equal(t.cpu().numpy().view(np.uint64), x)
    pb.scan(t, out=t, exclusive=exclusive)
    torch.cuda.synchronize()
    assert np.array_equal(t.cpu().numpy().view(np.uint64), want)


def test_scan_int64_large_with_carries_between_the_halves(pb):
    """2^26 elements just below 2^32 each: the running sum crosses 2^32 every element or two, so the low half of a
    tile's record overflows into the high half all the time; checked completely."""
    n = 1 << 26
    g = torch.Generator(device=DEV).manual_seed(64)
    x = torch.randint((1 << 32) - (1 << 20), 1 << 32, (n,), dtype=torch.int64, device=DEV, generator=g)
    out = pb.scan(x)
    torch.cuda.synchronize()
    assert torch.equal(out, torch.cumsum(x, 0))


def test_scan_int64_workspace_is_twice_the_uint32_one(pb):
    import ctypes
    import prism_b200._lib as L
    lib = L.load()
    a, b = ctypes.c_size_t(0), ctypes.c_size_t(0)
    assert lib.prism_b200_scan_general_workspace_size(1 << 20, 0, ctypes.byref(a)) == 0
    assert lib.prism_b200_scan_general_workspace_size(1 << 20, 4, ctypes.byref(b)) == 0
    assert a.value == pb.get_workspace_size(1 << 20) and b.value - 128 == 2 * (a.value - 128)
    x = torch.zeros(16, dtype=torch.int64, device=DEV)
    ws = torch.empty(b.value, dtype=torch.uint8, device=DEV)
    assert lib.prism_b200_scan_general(16, x.data_ptr(), x.data_ptr(), ws.data_ptr(), 2 | 4, None) == 1   # F32 and I64
    pb.clear_error()


def test_scan_general_rejects_partial_overlap(pb):
    buf = torch.zeros(4096 + 8, dtype=torch.int32, device=DEV)
    ws = pb.scan_workspace(4096, DEV)
    import prism_b200._lib as L
    rc = L.load().prism_b200_scan_general(4096, buf.data_ptr(), buf.data_ptr() + 16, ws.data_ptr(), 0, None)
    assert rc == 1 and "overlap" in pb.last_error()[1]
    pb.clear_error()


def test_scan_random_sizes_all_flavours(pb):
    """Thirty seeded random sizes up to 2^21 with full-range values: in place, separate output, exclusive."""
    rng = np.random.default_rng(57721)
    for _ in range(30):
        n = int(rng.integers(1, 1 << 21))
        x = rng.integers(0, 1 << 32, n, dtype=np.uint64).astype(np.uint32)
        inc = O.scan_cpu(x)
        t = torch.from_numpy(x.view(np.int32).copy()).to(DEV)
        ex = pb.scan(t, exclusive=True)
        out = pb.scan(t)
        pb.scan_(t)
        torch.cuda.synchronize()
        assert np.array_equal(t.cpu().numpy().view(np.uint32), inc), n
        assert np.array_equal(out.cpu().numpy().view(np.uint32), inc), n
        assert np.array_equal(ex.cpu().numpy().view(np.uint32), np.concatenate([np.zeros(1, np.uint32), inc[:-1]])), n


def test_scan_rejects_misaligned(pb):
    x = torch.zeros(1024, dtype=torch.int32, device=DEV)
    with pytest.raises(pb.PrismB200Error) as e:
        pb.launch_scan(1000, x[1:], pb.scan_workspace(1000, DEV))
    assert e.value.code == 3
    pb.clear_error()
