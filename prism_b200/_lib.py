"""ctypes binding of libprism_b200.so (the C ABI declared in include/prism_b200.h).

There is no fallback: if the shared library is missing and cannot be built, or a
call returns a non-zero status, an exception is raised.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_size_t, c_ulonglong, c_void_p, POINTER
from pathlib import Path

from . import build as _build

PKG_DIR = Path(__file__).resolve().parent

STATUS_NAMES = {
    0: "OK",
    1: "INVALID_ARGUMENT",
    2: "UNSUPPORTED_SHAPE",
    3: "MISALIGNED",
    4: "CUDA",
    5: "DEVICE_TIMEOUT",
    6: "TOO_LARGE",
}

# name -> (restype, argtypes); mirrors include/prism_b200.h one to one.
SIGNATURES = {
    "prism_b200_version": (c_int, []),
    "prism_b200_last_error": (c_int, [POINTER(c_int), c_char_p, c_size_t]),
    "prism_b200_clear_error": (None, []),
    "prism_b200_launch_count": (c_ulonglong, []),
    "prism_b200_selftest_wait_timeout": (c_int, [c_ulonglong, c_void_p]),
    "prism_b200_sgemm": (c_int, [c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_float, c_void_p, c_void_p]),
    "prism_b200_gemm_bf16_fill_mode": (c_int, [c_int]),
    "prism_b200_gemm_bf16_fill_plan": (c_int, [c_int, c_int, c_int, c_int, c_int, POINTER(c_int), POINTER(c_int)]),
    "prism_b200_sgemm_tile_mode": (c_int, [c_int]),
    "prism_b200_sgemm_k_slices": (c_int, [c_int]),
    "prism_b200_sgemm_plan": (c_int, [c_int, c_int, c_int, c_int, POINTER(c_int), POINTER(c_int)]),
    "prism_b200_scan_workspace_size": (c_int, [c_size_t, POINTER(c_size_t)]),
    "prism_b200_scan": (c_int, [c_size_t, c_void_p, c_void_p, c_void_p]),
    "prism_b200_scan_f32": (c_int, [c_size_t, c_void_p, c_void_p, c_void_p]),
    "prism_b200_scan_general": (c_int, [c_size_t, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "prism_b200_scan_general_workspace_size": (c_int, [c_size_t, c_int, POINTER(c_size_t)]),
    "prism_b200_reduce_u32": (c_int, [c_size_t, c_void_p, c_void_p, c_void_p]),
    "prism_b200_scan_seeded": (c_int, [c_size_t, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "prism_b200_scan_add_carry": (c_int, [c_size_t, c_void_p, c_void_p, c_int, c_void_p]),
    "prism_b200_scan_publish_total": (c_int, [c_void_p, c_void_p, c_int, c_int, ctypes.c_uint32, c_void_p]),
    "prism_b200_scan_seeded_peers": (c_int, [c_size_t, c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.c_uint32, c_void_p]),
    "prism_b200_scan_sharded": (c_int, [c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.c_uint32, c_int,
                                        c_ulonglong, c_void_p]),
    "prism_b200_scan_static": (c_int, [c_size_t, c_void_p, c_void_p]),
    "prism_b200_gemm_bf16": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "prism_b200_gemm_bf16_axpby": (c_int, [c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p]),
    "prism_b200_peer_push": (c_int, [c_void_p, c_size_t, c_void_p, c_size_t, c_int, c_int, c_void_p, c_int, ctypes.c_uint32, c_void_p, c_void_p]),
    "prism_b200_peer_wait": (c_int, [c_void_p, c_int, c_int, ctypes.c_uint32, c_ulonglong, c_void_p]),
    "prism_b200_host_gemm_bf16_create": (c_int, [c_int, c_int, c_int, c_int, POINTER(c_void_p)]),
    "prism_b200_host_gemm_bf16_run": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "prism_b200_host_sgemm_create": (c_int, [c_int, c_int, c_int, c_int, c_int, POINTER(c_void_p)]),
    "prism_b200_host_sgemm_run": (c_int, [c_void_p, c_float, c_void_p, c_void_p, c_float, c_void_p, c_void_p]),
    "prism_b200_host_scan_create": (c_int, [c_size_t, c_size_t, POINTER(c_void_p)]),
    "prism_b200_host_scan_run": (c_int, [c_void_p, c_void_p, c_void_p]),
    "prism_b200_host_plan_blocks": (c_int, [c_void_p]),
    "prism_b200_host_plan_destroy": (None, [c_void_p]),
}


class PrismB200Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"prism_b200 status {code} ({STATUS_NAMES.get(code, '?')}): {message}")
        self.code = code
        self.message = message


_lib = None


def lib_path() -> Path:
    return _build.LIB_PATH


def load(build_if_missing: bool = True) -> ctypes.CDLL:
    """Load (building first if needed) the shared library and type its entry points."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    if _build.stale():
        # A library built from other sources than the ones in the tree is never loaded silently.
        if not build_if_missing:
            raise FileNotFoundError(f"{path} is missing or older than its sources; run `python -m prism_b200.build`")
        _build.build_library()
    lib = ctypes.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> tuple[int, str]:
    lib = load()
    code = c_int(0)
    buf = ctypes.create_string_buffer(256)
    lib.prism_b200_last_error(ctypes.byref(code), buf, 256)
    return code.value, buf.value.decode(errors="replace")


def check(status: int) -> None:
    if status != 0:
        _, msg = last_error()
        raise PrismB200Error(status, msg)
