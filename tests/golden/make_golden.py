"""Writes tests/golden/scan_ref_cpu.npz from the reference's own CPU scan loop.

    python oracle/build_ref.py && python tests/golden/make_golden.py

Needs oracle/_ref/libref_cpu.so, i.e. the reference tree at build time
(scan_cpu, evals/4090_scan/scan_harness.cuh:30-36, compiled where it lies).
Inputs are seeded; sizes are small so the fixture stays a few hundred KB.
"""
import ctypes
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import cpu_oracle as O  # noqa: E402


def main():
    lib = ctypes.CDLL(str(ROOT / "oracle" / "_ref" / "libref_cpu.so"))
    lib.ref_scan_cpu.argtypes = [ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p]
    cases = {
        "small": O.scan_inputs(100, seed=1, high=101),                 # the harness's value range
        "tile": O.scan_inputs(16384, seed=2, high=16),                 # one reference tile, config #2 values
        "ragged": O.scan_inputs(16384 + 4096 + 37, seed=3, high=2),    # not a multiple of any tile
        "wrap": O.scan_inputs(20000, seed=4, high=0xFFFFFFFF),         # 32-bit wrap-around
    }
    out = {}
    for name, x in cases.items():
        y = np.empty_like(x)
        lib.ref_scan_cpu(x.size, x.ctypes.data_as(ctypes.c_void_p), y.ctypes.data_as(ctypes.c_void_p))
        out[name + "_in"], out[name + "_out"] = x, y
    np.savez_compressed(ROOT / "tests" / "golden" / "scan_ref_cpu.npz", **out)
    print("wrote", ROOT / "tests" / "golden" / "scan_ref_cpu.npz")


if __name__ == "__main__":
    main()
