"""Readers for the three line formats that the evaluation programs print, written after what the reference's
plotting script extracts from them (evals/plot_results.py:18-108): per bf16 size a `Kernel:` line followed by a
`cuBLAS:` line; per SGEMM size a `Size: AxBxC` heading, `[cuBLAS FP32]` / `[My Kernel k]` headings and one
`performance: (x) GFLOPS` line each, after the `Starting Performance Sweep` banner; and the scan table of
`size | cub_ms cub_gbs | ours_ms ours_gbs` rows under its header.  tests/golden/evals_parsed_by_reference.json
holds what the reference's own script returned for the committed sample outputs, and tests/test_evals_format.py
checks that these readers return the same."""
import re

SGEMM_NAMES = {1: "Naive", 2: "Mem Coalescing", 3: "2D SMEM Tiling", 4: "2D Tiling + Vectorize", 5: "Warp Tiling"}
_RATE = r"performance:\s+\(\s*([\d.]+)\)\s+%s.*size:\s+\((\d+)\)"


def bf16_rows(text):
    """[(size, kernel TFLOP/s, cuBLAS TFLOP/s)]: a cuBLAS line closes the Kernel line before it."""
    rows, ours = [], None
    for line in text.splitlines():
        k = re.search(r"Kernel:\s+.*" + _RATE % "TFLOPS", line)
        if k:
            ours = float(k.group(1))
        c = re.search(r"cuBLAS:\s+.*" + _RATE % "TFLOPS", line)
        if c and ours is not None:
            rows.append((int(c.group(2)), ours, float(c.group(1))))
            ours = None
    return rows


def sgemm_rows(text):
    """{kernel name: [(size, GFLOP/s)]} from the part after the sweep banner."""
    out = {}
    _, banner, sweep = text.partition("Starting Performance Sweep")
    if not banner:
        return out
    size = name = None
    for raw in sweep.splitlines():
        line = raw.strip()
        m = re.match(r"Size:\s+(\d+)x(\d+)x(\d+)", line)
        if m:
            size = int(m.group(1))
            continue
        if size is None:
            continue
        if line.startswith("[cuBLAS FP32]"):
            name = "cuBLAS"
            continue
        m = re.match(r"\[My Kernel (\d+)\]", line)
        if m:
            k = int(m.group(1))
            name = SGEMM_NAMES.get(k, f"Kernel {k}")
            continue
        m = re.search(_RATE % "GFLOPS", raw)
        if m and name:
            out.setdefault(name, []).append((size, float(m.group(1))))
            name = None
    return out


def scan_rows(text):
    """[(n, CUB GB/s, ours GB/s)] from the table that starts at the header naming `CUB (GB/s)`."""
    rows, inside = [], False
    for raw in text.splitlines():
        line = raw.strip()
        if "Size" in raw and "CUB (GB/s)" in raw:
            inside = True
        elif inside and not line:
            inside = False
        elif inside and not line.startswith("---"):
            cells = re.split(r"\s*\|\s*", line)
            try:
                rows.append((int(cells[0]), float(cells[1].split()[1]), float(cells[2].split()[1])))
            except (ValueError, IndexError):
                pass
    return rows
