"""How the 512 x 256 form of the bf16 GEMM deals its work to the CTA pairs (prism_b200_gemm_bf16_fill_plan: the
function the kernel itself evaluates, compiled for the host too).  Checked without a GPU: every tile is computed
exactly once -- whole, or as each of its two n blocks once -- only tiles of the last, partly filled wave are cut,
pieces come after a pair's whole tiles, and no pair gets more than its share of pieces."""
import ctypes
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def _items(lib, tiles, pairs, fill, pair):
    count = ctypes.c_int()
    assert lib.prism_b200_gemm_bf16_fill_plan(tiles, pairs, fill, pair, 0, None, ctypes.byref(count)) == 0
    buf = (ctypes.c_int * (2 * max(count.value, 1)))()
    assert lib.prism_b200_gemm_bf16_fill_plan(tiles, pairs, fill, pair, count.value, buf, ctypes.byref(count)) == 0
    return [(buf[2 * i], buf[2 * i + 1]) for i in range(count.value)]


# (tiles, pairs): the benchmark shape on 1, 2, 4 and 8 GPUs, 4096^3, 6144^3, 12288^3, corner cases
CASES = [(512, 74), (256, 74), (128, 74), (64, 74), (288, 74), (1152, 74), (1, 74), (1, 2), (73, 74), (74, 74), (75, 74),
         (148, 74), (3, 4), (5, 3), (1, 3), (0, 74), (19, 74), (37, 74), (38, 74)]


@pytest.mark.parametrize("tiles,pairs", CASES)
@pytest.mark.parametrize("fill", [0, 1])
def test_every_tile_is_computed_once(tiles, pairs, fill):
    from prism_b200 import _lib
    lib = _lib.load()
    full, rem = divmod(tiles, pairs)
    whole, pieces, most = set(), set(), 0
    for p in range(pairs):
        items = _items(lib, tiles, pairs, fill, p)
        mine = 0
        for i, (t, blk) in enumerate(items):
            assert 0 <= t < tiles
            if blk < 0:
                assert t not in whole and t == i * pairs + p
                assert not fill or t < full * pairs            # with a fill, whole tiles only in the full waves
                whole.add(t)
            else:
                assert fill and blk in (0, 1) and t >= full * pairs and (t, blk) not in pieces
                assert all(b >= 0 for _, b in items[i:])       # pieces come after the whole tiles
                pieces.add((t, blk))
                mine += 1
        most = max(most, mine)
    if not fill:
        assert whole == set(range(tiles)) and not pieces
    else:
        assert whole == set(range(full * pairs))
        assert pieces == {(t, b) for t in range(full * pairs, tiles) for b in (0, 1)}
        assert most == -(-rem * 2 // pairs)


def test_argument_checks():
    from prism_b200 import _lib
    lib = _lib.load()
    n = ctypes.c_int()
    assert lib.prism_b200_gemm_bf16_fill_plan(8, 4, 2, 0, 0, None, ctypes.byref(n)) == 1     # fill is 0 or 1
    assert lib.prism_b200_gemm_bf16_fill_plan(8, 4, 1, 4, 0, None, ctypes.byref(n)) == 1     # pair outside
    assert lib.prism_b200_gemm_bf16_fill_plan(8, 4, 1, 0, 4, None, ctypes.byref(n)) == 1     # room but no array
    assert lib.prism_b200_gemm_bf16_fill_mode(4) == 1
    lib.prism_b200_clear_error()
