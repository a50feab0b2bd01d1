"""The output of this repository's evaluation programs is what the reference's plotting script reads
(evals/plot_results.py:18-108).  tests/golden/evals_output_b200/ holds their output from a B200 (SGEMM sweep at the
reference's six sizes, scan table 2^20 ... 2^30, bf16 sweep 2048 ... 16384) and
tests/golden/evals_parsed_by_reference.json what the reference's own parse functions returned for it
(tests/golden/make_evals_parse.py).  Here: the readers that the GPU tests use on fresh output (tests/evals_lines.py)
return exactly that, the samples are complete sweeps, and -- where a checkout of the reference is at hand -- the
reference's functions are run again on the samples."""
import json
import os
import sys
from pathlib import Path

import pytest

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
sys.path.insert(0, str(HERE / "golden"))
import evals_lines as L  # noqa: E402
import make_evals_parse as G  # noqa: E402

SAMPLES = HERE / "golden" / "evals_output_b200"
EXPECT = json.loads((HERE / "golden" / "evals_parsed_by_reference.json").read_text())


def _as_lists(rows):
    return [list(r) for r in rows]


def test_bf16_lines_read_like_the_reference_script():
    got = L.bf16_rows((SAMPLES / "bf16_bench.txt").read_text())
    assert _as_lists(got) == EXPECT["bf16"]
    assert [r[0] for r in got] == [2048, 4096, 6144, 8192, 12288, 16384]          # evals/run_h100.sh:12
    assert all(k > 0 and c > 0 for _, k, c in got)


def test_sgemm_lines_read_like_the_reference_script():
    got = L.sgemm_rows((SAMPLES / "sgemm_sweep.txt").read_text())
    assert {k: _as_lists(v) for k, v in got.items()} == EXPECT["sgemm"]
    assert set(got) == {"cuBLAS", *L.SGEMM_NAMES.values()}
    for rows in got.values():
        assert [s for s, _ in rows] == [256, 512, 1024, 2048, 4096, 8192]          # evals/4090_sgemm/main.cu sweep


def test_scan_table_reads_like_the_reference_script():
    got = L.scan_rows((SAMPLES / "scan_bench.txt").read_text())
    assert _as_lists(got) == EXPECT["scan"]
    assert [n for n, _, _ in got] == [1 << p for p in range(20, 31)]               # evals/4090_scan/main.cu:96-128


def test_readers_skip_what_the_reference_script_skips():
    text = ("Size | CUB (ms) CUB (GB/s) | Ours (ms) Ours (GB/s)\n---+---+---\n1024 | 0.1 10.0 | 0.2 5.0\nbad | x | y\n"
            "2048 | 0.1 | 0.2 7.0\n\n4096 | 0.1 1.0 | 0.1 1.0\n")
    assert L.scan_rows(text) == [(1024, 10.0, 5.0)]            # malformed rows dropped, a blank line ends the table
    pre = "[My Kernel 5]\nAverage elapsed time: (0.1) s, performance: ( 9.9) GFLOPS. size: (64).\n"
    assert L.sgemm_rows(pre) == {}                              # nothing counts before the sweep banner
    text = pre + "Starting Performance Sweep\nSize: 64x64x64\n[My Kernel 7]\n" + pre.splitlines()[1] + "\n"
    assert L.sgemm_rows(text) == {"Kernel 7": [(64, 9.9)]}
    assert L.bf16_rows("cuBLAS:  Average elapsed time: (1) s, performance: ( 1.0) TFLOPS. size: (64).\n") == []


def test_reference_script_itself_on_the_samples():
    root = os.environ.get("PRISM_REFERENCE", str(HERE.parent.parent / "reference"))
    mod = G.load_reference_parser(root)
    if mod is None:
        pytest.skip("no checkout of the reference (set PRISM_REFERENCE)")
    assert G.parse_samples(mod) == EXPECT
