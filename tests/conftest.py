import ctypes
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def _has_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle_c():
    """The plain-C restatement (oracle/oracle_cpu.c), built on demand."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import build_ref
    lib = ctypes.CDLL(str(build_ref.build_oracle_c()))
    lib.oracle_scan_u32.argtypes = [ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p]
    lib.oracle_sgemm_f32.argtypes = [ctypes.c_int] * 3 + [ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p,
                                                          ctypes.c_float, ctypes.c_void_p]
    lib.oracle_gemm_bf16.argtypes = [ctypes.c_int] * 3 + [ctypes.c_void_p] * 3
    return lib


@pytest.fixture(scope="session")
def ref_cpu():
    """The reference's own CPU scan loop, if oracle/_ref was built (needs the reference tree at build time)."""
    p = ROOT / "oracle" / "_ref" / "libref_cpu.so"
    if not p.exists():
        pytest.skip("oracle/_ref/libref_cpu.so not built (reference tree absent)")
    lib = ctypes.CDLL(str(p))
    lib.ref_scan_cpu.argtypes = [ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p]
    return lib


@pytest.fixture(scope="session")
def ref_gpu():
    """The reference's generated kernels recompiled for sm_100 (oracle/_ref/libprism_ref.so)."""
    p = ROOT / "oracle" / "_ref" / "libprism_ref.so"
    if not p.exists():
        pytest.skip("oracle/_ref/libprism_ref.so not built (reference tree absent)")
    lib = ctypes.CDLL(str(p))
    lib.ref_sgemm.argtypes = [ctypes.c_int] * 4 + [ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float,
                                                   ctypes.c_void_p]
    lib.ref_sgemm.restype = ctypes.c_int
    lib.ref_scan_workspace_size.argtypes = [ctypes.c_size_t]
    lib.ref_scan_workspace_size.restype = ctypes.c_size_t
    lib.ref_scan.argtypes = [ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p]
    lib.ref_scan.restype = ctypes.c_int
    return lib


@pytest.fixture(scope="session")
def pb():
    import prism_b200
    prism_b200.load()
    return prism_b200


@pytest.fixture(autouse=True)
def _no_sticky_error(request):
    """A GPU test must leave no device-side timeout behind."""
    yield
    if "gpu" in request.keywords and _has_gpu():
        import torch
        import prism_b200
        torch.cuda.synchronize()
        code, msg = prism_b200.last_error()
        prism_b200.clear_error()
        assert code in (0, 1, 2, 3, 6), f"device/runtime error left behind: {code} {msg}"
