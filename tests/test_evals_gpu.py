"""The evaluation programs (prism_b200/evals) on small sizes: they must pass their own checks against
cuBLAS / CUB / a CPU loop and print lines in the formats the reference's plotting script parses
(evals/plot_results.py:18-108).  The lines are read with tests/evals_lines.py, which tests/test_evals_format.py
pins to what the reference's own script returns on sample outputs."""
import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(Path(__file__).resolve().parent))
import evals_lines as L  # noqa: E402

EVALS = ROOT / "prism_b200" / "evals"
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def binaries():
    sys.path.insert(0, str(ROOT))
    from prism_b200 import build
    build.build_library()
    build.build_evals()
    return EVALS / "build"


def _run(cmd):
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return r.stdout


def test_sgemm_sweep_format_and_checks(binaries):
    out = _run([binaries / "sgemm_sweep", 512])
    assert out.count("PASSED") == 5 and "FAILED" not in out
    perf = out.split("Starting Performance Sweep")[1]
    sizes = [int(m.group(1)) for m in re.finditer(r"^Size:\s+(\d+)x(\d+)x(\d+)", perf, re.M)]
    assert sizes == [256, 512]
    assert len(re.findall(r"^\[cuBLAS FP32\]", perf, re.M)) == 2
    assert [int(k) for k in re.findall(r"^\[My Kernel (\d+)\]", perf, re.M)] == [1, 2, 3, 4, 5] * 2
    vals = re.findall(r"performance:\s+\(\s*([\d.]+)\)\s+GFLOPS.*size:\s+\((\d+)\)", perf)
    assert len(vals) == 12 and all(float(v) > 0 for v, _ in vals)
    rows = L.sgemm_rows(out)
    assert set(rows) == {"cuBLAS", *L.SGEMM_NAMES.values()}
    assert all([s for s, _ in r] == [256, 512] and all(g > 0 for _, g in r) for r in rows.values())


def test_scan_bench_format_and_checks(binaries):
    out = _run([binaries / "scan_bench", 21])
    assert "mismatch" not in out
    lines = out.strip().splitlines()
    assert "Size" in lines[0] and "CUB (GB/s)" in lines[0] and lines[1].startswith("---")
    rows = L.scan_rows(out)
    assert len(rows) == len(lines) - 2 and [r[0] for r in rows] == [1 << 20, 1 << 21]
    assert all(cub > 0 and ours > 0 for _, cub, ours in rows)


def test_bf16_bench_format_and_checks(binaries):
    out = _run([binaries / "bf16_bench", 1024])
    assert "Passed correctness verification!" in out
    k = re.search(r"Kernel:\s+.*performance:\s+\(\s*([\d.]+)\)\s+TFLOPS.*size:\s+\((\d+)\)", out)
    c = re.search(r"cuBLAS:\s+.*performance:\s+\(\s*([\d.]+)\)\s+TFLOPS.*size:\s+\((\d+)\)", out)
    assert k and c and int(k.group(2)) == 1024 and float(k.group(1)) > 0 and float(c.group(1)) > 0
    assert L.bf16_rows(out) == [(1024, float(k.group(1)), float(c.group(1)))]


def test_reference_sgemm_sweep_relinked_against_this_library():
    """The reference's own sweep program (evals/4090_sgemm/main.cu, compiled unmodified where a checkout of the
    reference was present) linked against this library instead of its runner.cu: its cuBLAS comparison must pass
    for kernels 1-5 and the sweep must print all six sizes.  Skipped where the binary was not built."""
    exe = ROOT / "oracle" / "_ref" / "relink_sgemm_sweep"
    if not exe.exists():
        pytest.skip("oracle/_ref/relink_sgemm_sweep not built (needs a checkout of the reference at build time)")
    out = _run([exe])
    assert out.count("Correctness: PASSED") == 5 and "Divergence" not in out
    perf = out.split("Starting Performance Sweep")[1]
    sizes = [int(m.group(1)) for m in re.finditer(r"^Size:\s+(\d+)x(\d+)x(\d+)", perf, re.M)]
    assert sizes == [256, 512, 1024, 2048, 4096, 8192]
    vals = re.findall(r"performance:\s+\(\s*([\d.]+)\)\s+GFLOPS.*size:\s+\((\d+)\)", perf)
    assert len(vals) == 36 and all(float(v) > 0 for v, _ in vals)


def test_reference_scan_harness_relinked_against_this_library():
    """The reference's scan harness program (evals/4090_scan/main.cu with scan_harness.cuh, both unmodified,
    compiled where a checkout of the reference was present) on this library's scan: its own element-by-element
    comparison with scan_cpu must pass at its five sizes (16384 ... 64 Mi) and its benchmark must print a
    throughput.  Skipped where the binary was not built."""
    exe = ROOT / "oracle" / "_ref" / "relink_scan_main"
    if not exe.exists():
        pytest.skip("oracle/_ref/relink_scan_main not built (needs a checkout of the reference at build time)")
    out = _run([exe])
    assert "Mismatch" not in out and "not yet implemented" not in out
    sizes = [int(m.group(1)) for m in re.finditer(r"Testing size\s+(\d+)", out)]
    assert sizes == [16384, 32768, 1 << 20, 16 << 20, 64 << 20]
    assert out.count("  OK") == 5
    m = re.search(r"Throughput:\s+([\d.]+) GB/s", out)
    assert m and float(m.group(1)) > 0


def test_reference_bf16_benchmark_relinked_against_this_library():
    """The reference's bf16 benchmark program (evals/h100_bench/main.cu, unmodified, compiled where a checkout of the
    reference was present, with a stand-in for its Hopper-only utils.cuh that routes runmyh100 to this library):
    its own comparison with cuBLAS (0.1 absolute on normal(0, 1) inputs) must pass at 2048 and at its default size
    6144, and its two result lines must read the way the reference's plotting script reads them."""
    exe = ROOT / "oracle" / "_ref" / "relink_h100_main"
    if not exe.exists():
        pytest.skip("oracle/_ref/relink_h100_main not built (needs a checkout of the reference at build time)")
    for args, size in (([2048], 2048), ([], 6144)):
        out = _run([exe, *args])
        assert "Testing prism_h100::runmyh100" in out and "Passed correctness verification!" in out
        assert "Divergence" not in out and "Failed" not in out
        rows = L.bf16_rows(out)
        assert len(rows) == 1 and rows[0][0] == size and rows[0][1] > 0 and rows[0][2] > 0


def test_host_e2e_program_through_the_c_abi_alone(binaries):
    """Host plans driven from C++ with cudaHostAlloc'ed arrays (no Python on the data path), small sizes."""
    out = _run([binaries / "host_e2e", 1024, 512, 23])
    assert out.strip().endswith("PASSED") and "mismatch" not in out
    assert len(re.findall(r"^host (bf16 GEMM|SGEMM|scan) .* end to end", out, re.M)) == 3
