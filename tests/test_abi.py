"""The C-ABI library: it loads, exports every symbol the header declares, and its
host-side argument checks answer without touching a GPU."""
import ctypes
import re
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from prism_b200 import _lib, build  # noqa: E402


def declared_symbols():
    text = (ROOT / "include" / "prism_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(prism_b200_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for must in ("prism_b200_sgemm", "prism_b200_scan", "prism_b200_scan_workspace_size", "prism_b200_gemm_bf16",
                 "prism_b200_last_error", "prism_b200_version"):
        assert must in names


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build_library()
    lib = ctypes.CDLL(str(path))
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in include/prism_b200.h but not exported"


def test_python_binding_covers_every_declared_symbol():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_version():
    assert _lib.load().prism_b200_version() >= 100


def test_workspace_size_is_host_only_and_monotonic():
    lib = _lib.load()
    out = ctypes.c_size_t(0)
    sizes = []
    for n in (0, 1, 4096, 4097, 1 << 24, 1 << 28, 1 << 30):
        assert lib.prism_b200_scan_workspace_size(n, ctypes.byref(out)) == 0
        sizes.append(out.value)
    assert sizes == sorted(sizes) and sizes[0] > 0
    # one record (a 32-byte sector) per 4096-element tile plus a 128-byte header
    assert sizes[4] == 128 + ((1 << 24) // 4096) * 32


def test_argument_errors_are_reported_not_fatal():
    lib = _lib.load()
    lib.prism_b200_clear_error()
    assert lib.prism_b200_sgemm(9, 128, 128, 128, 1.0, None, None, 0.0, None, None) == 1
    code, msg = _lib.last_error()
    assert code == 1 and "kernel id" in msg
    assert lib.prism_b200_sgemm(5, -1, 128, 128, 1.0, None, None, 0.0, None, None) == 1
    out = ctypes.c_size_t(0)
    assert lib.prism_b200_scan_workspace_size(1 << 32, ctypes.byref(out)) == 6
    assert lib.prism_b200_scan_workspace_size(16, None) == 1
    assert lib.prism_b200_gemm_bf16(100, 128, 64, None, None, None, None) == 1   # null pointers first
    assert lib.prism_b200_gemm_bf16(-1, 128, 64, None, None, None, None) == 1
    assert lib.prism_b200_scan(0, None, None, None) == 0                         # empty input is a no-op
    assert lib.prism_b200_sgemm(5, 0, 128, 128, 1.0, None, None, 0.0, None, None) == 0
    lib.prism_b200_clear_error()
    assert _lib.last_error()[0] == 0


def test_no_cpu_fallback_in_python_layer():
    import torch
    import prism_b200 as pb
    x = torch.zeros(16, dtype=torch.int32)
    with pytest.raises(TypeError):
        pb.scan_(x)
    with pytest.raises(TypeError):
        pb.sgemm(torch.zeros(2, 2), torch.zeros(2, 2), torch.zeros(2, 2))


def test_package_does_not_import_the_oracle():
    for py in (ROOT / "prism_b200").rglob("*.py"):
        assert "oracle" not in py.read_text(), py
    for cu in (ROOT / "prism_b200" / "csrc").iterdir():
        assert "oracle" not in cu.read_text(), cu
