"""The division of the bf16 GEMM's last, partly filled wave of tiles among the CTA pairs
(prism_b200_gemm_bf16_split_plan: the function the kernel itself evaluates, compiled for the host too).
Checked without a GPU: every (tile, k-block) is computed exactly once, every tile has exactly one pair
that holds its k-block 0, contributions come first in a pair's order and the finishing segment last."""
import ctypes
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def _plans(lib, tiles, pairs, kb):
    out = (ctypes.c_int * 7)()
    plans = []
    for p in range(pairs):
        assert lib.prism_b200_gemm_bf16_split_plan(tiles, pairs, kb, p, out) == 0
        plans.append(list(out))
    return plans


# (tiles, pairs, k_blocks): the benchmark shape on 1, 2, 4 and 8 GPUs, 4096^3, 6144^3, 12288^3, and corner cases
CASES = [(512, 74, 128), (256, 74, 128), (128, 74, 128), (64, 74, 128), (128, 74, 64), (288, 74, 96), (1152, 74, 192),
         (1, 74, 128), (73, 74, 5), (75, 74, 1), (3, 4, 2), (148, 74, 7), (5, 3, 4), (1, 3, 2)]


@pytest.mark.parametrize("tiles,pairs,kb", CASES)
def test_every_k_block_of_every_tile_is_computed_once(tiles, pairs, kb):
    from prism_b200 import _lib
    lib = _lib.load()
    seen = {}
    heads = {}
    for p, (full, segs, t0, a0, b0, t1, b1) in enumerate(_plans(lib, tiles, pairs, kb)):
        assert full == tiles // pairs and 0 <= segs <= 2
        items = [(i * pairs + p, 0, kb) for i in range(full)]
        if segs >= 1:
            items.append((t0, a0, b0))
        if segs == 2:
            assert t1 == t0 + 1 and a0 > 0, "a second segment is the head of the next tile, after a tail"
            items.append((t1, 0, b1))
        for t, a, b in items:
            assert 0 <= t < tiles and 0 <= a < b <= kb
            for k in range(a, b):
                assert (t, k) not in seen, f"tile {t} k-block {k} computed by pairs {seen[(t, k)]} and {p}"
                seen[(t, k)] = p
            if a == 0:
                assert t not in heads
                heads[t] = p
    assert len(seen) == tiles * kb
    assert sorted(heads) == list(range(tiles))
    # the pairs that complete a tile follow its finisher in pair order, without a gap
    for t in range(tiles):
        owners = sorted({seen[(t, k)] for k in range(kb)})
        assert owners[0] == heads[t] and owners == list(range(owners[0], owners[-1] + 1))
