"""Which tile and how many CTAs per tile along K the launcher of SGEMM kernel 5 takes (prism_b200_sgemm_plan: the
function the launcher itself evaluates), checked without a GPU against the forms that measured best, or within 1 % of
the best, on a B200 with 148 SMs (back-to-back launches, every candidate forced in turn)."""
import ctypes
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def _plan(lib, M, N, K, sms=148):
    tile, slices = ctypes.c_int(-9), ctypes.c_int(-9)
    assert lib.prism_b200_sgemm_plan(M, N, K, sms, ctypes.byref(tile), ctypes.byref(slices)) == 0
    return tile.value, slices.value


# shape -> the candidates (tile, slices) that measured best or within 1 % of it
MEASURED = {
    (256, 256, 256): {(2, 4), (2, 2), (1, 4)},
    (512, 512, 512): {(1, 4)},
    (768, 768, 768): {(1, 2)},
    (1024, 1024, 1024): {(1, 2), (1, 4)},
    (1280, 1280, 1280): {(1, 2)},
    (1536, 1536, 1536): {(0, 1), (1, 2)},
    (2048, 2048, 2048): {(1, 2)},
    (3072, 3072, 3072): {(0, 1)},
    (4096, 4096, 4096): {(0, 1)},
    (128, 4096, 4096): {(1, 4)},
    (256, 4096, 4096): {(1, 4)},
    (512, 4096, 4096): {(1, 2), (1, 4)},
    (1024, 4096, 4096): {(1, 2)},
    (2048, 4096, 4096): {(1, 1), (1, 2)},
    (512, 512, 4096): {(1, 4)},
    (1024, 1024, 4096): {(1, 4)},
}


@pytest.mark.parametrize("shape", sorted(MEASURED))
def test_launcher_takes_a_form_that_measured_best(shape):
    from prism_b200 import _lib
    assert _plan(_lib.load(), *shape) in MEASURED[shape]


def test_switches_and_shapes_the_tiles_do_not_divide():
    from prism_b200 import _lib
    lib = _lib.load()
    assert _plan(lib, 8192, 8192, 8192) == (0, 1)
    assert _plan(lib, 1000, 1024, 1024) == (-1, 1) and _plan(lib, 1024, 1024, 1000) == (-1, 1)
    assert _plan(lib, 1024, 1024, 1040)[1] == 1                 # 1040 = 16 * 65: no sharing divides K
    assert _plan(lib, 1024, 1024, 1056)[1] in (1, 2)            # 1056 = 16 * 66: two CTAs at most
    try:
        assert lib.prism_b200_sgemm_k_slices(1) == 0
        assert all(_plan(lib, *shape)[1] == 1 for shape in MEASURED)
        assert _plan(lib, 1024, 1024, 1024) == (1, 1) and _plan(lib, 4096, 4096, 4096) == (0, 1)
        assert lib.prism_b200_sgemm_k_slices(4) == 0
        assert _plan(lib, 1024, 1024, 1056)[1] == 2 and _plan(lib, 1024, 1024, 1040)[1] == 1
        assert lib.prism_b200_sgemm_tile_mode(2) == 0
        assert _plan(lib, 4096, 4096, 4096) == (2, 4)
        assert lib.prism_b200_sgemm_tile_mode(0) == 0
        assert _plan(lib, 1024, 1024, 1024) == (0, 1)            # 128 x 128 tiles are never shared
    finally:
        lib.prism_b200_sgemm_tile_mode(-1)
        lib.prism_b200_sgemm_k_slices(-1)
    none = ctypes.c_int()
    assert lib.prism_b200_sgemm_plan(0, 128, 16, 148, ctypes.byref(none), ctypes.byref(none)) == 1
    assert lib.prism_b200_sgemm_plan(128, 128, 16, 148, None, ctypes.byref(none)) == 1
    lib.prism_b200_clear_error()
