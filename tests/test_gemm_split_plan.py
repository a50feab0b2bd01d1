"""How the bf16 GEMM shares its last, partly filled wave of tiles between the pairs that own a tile and the
pairs that would idle (prism_b200_gemm_bf16_split_plan: the function the kernel itself evaluates, compiled for
the host too).  Checked without a GPU: every (tile, k-block) is computed exactly once, every tile of the last
wave has one owner (k-blocks from 0) and one helper (the tail), and no helper has more than its share of tails."""
import ctypes
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def _plans(lib, tiles, pairs, kb, tail):
    out = (ctypes.c_int * 5)()
    plans = []
    for p in range(pairs):
        assert lib.prism_b200_gemm_bf16_split_plan(tiles, pairs, kb, tail, p, out) == 0
        plans.append(list(out))
    return plans


# (tiles, pairs, k_blocks, tail): the benchmark shape on 1, 2, 4 and 8 GPUs, 4096^3, 6144^3, 12288^3, corner cases
CASES = [(512, 74, 128, 6), (256, 74, 128, 62), (128, 74, 128, 29), (64, 74, 128, 12), (128, 74, 64, 13), (288, 74, 96, 20),
         (1152, 74, 192, 30), (1, 74, 128, 60), (73, 74, 5, 1), (75, 74, 3, 2), (3, 4, 2, 1), (148, 74, 7, 3), (5, 3, 4, 1),
         (1, 3, 2, 1), (74, 74, 16, 5)]


@pytest.mark.parametrize("tiles,pairs,kb,tail", CASES)
def test_every_k_block_of_every_tile_is_computed_once(tiles, pairs, kb, tail):
    from prism_b200 import _lib
    lib = _lib.load()
    full, rem = divmod(tiles, pairs)
    seen, owner, helper, tails_of = {}, {}, {}, {}
    for p, (f, segs, first, a, b) in enumerate(_plans(lib, tiles, pairs, kb, tail)):
        assert f == full
        items = [(i * pairs + p, 0, kb) for i in range(f)] + [(first + j, a, b) for j in range(segs)]
        for t, k0, k1 in items:
            assert 0 <= t < tiles and 0 <= k0 < k1 <= kb
            for k in range(k0, k1):
                assert (t, k) not in seen, f"tile {t} k-block {k} computed by pairs {seen[(t, k)]} and {p}"
                seen[(t, k)] = p
            if t >= full * pairs:
                if k0 == 0:
                    assert t not in owner and p < rem and t == full * pairs + p and k1 == kb - tail
                    owner[t] = p
                else:
                    assert t not in helper and p >= rem and (k0, k1) == (kb - tail, kb)
                    helper[t] = p
                    tails_of[p] = tails_of.get(p, 0) + 1
    assert len(seen) == tiles * kb
    last_wave = list(range(full * pairs, tiles))
    assert sorted(owner) == last_wave
    if rem:
        assert sorted(helper) == last_wave
        helpers = pairs - rem
        assert max(tails_of.values()) <= -(-rem // helpers) and len(tails_of) <= helpers
