"""The allocation-free scan entry point, prism_b200_scan_static.

It exists for callers that cannot allocate device memory where the scan runs
(plugins working only on buffers their host application owns, loops that must not
block on the allocator, processes whose device memory is all handed out): its
look-back records live in a fixed array inside the library instead of in
caller-provided scratch.  The test drives it through the C ABI twice in a row --
the second call finds the first call's records still in the array -- and requires
the same bits as prism_b200_scan and as the CPU oracle.
"""
import ctypes
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from oracle import cpu_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _abi():
    from prism_b200 import _lib
    return _lib.load(), _lib


def test_static_scan_matches_scan_on_two_calls_in_a_row():
    lib, _lib = _abi()
    stream = ctypes.c_void_p(torch.cuda.current_stream(torch.device(DEV)).cuda_stream)
    with torch.cuda.device(DEV):
        for call, (n, high, seed) in enumerate([((1 << 22) + 12345, 1 << 20, 1), ((1 << 20) + 3, 16, 2)]):
            g = torch.Generator(device=DEV).manual_seed(seed)
            src = torch.randint(0, high, (n,), dtype=torch.int32, device=DEV, generator=g)
            # existing entry point, caller-provided scratch
            size = ctypes.c_size_t(0)
            assert lib.prism_b200_scan_workspace_size(n, ctypes.byref(size)) == 0
            ws = torch.empty(size.value, dtype=torch.uint8, device=DEV)
            want = src.clone()
            assert lib.prism_b200_scan(n, want.data_ptr(), ws.data_ptr(), stream) == 0
            # allocation-free entry point; the second pass reuses the array the first one left behind
            got = src.clone()
            torch.cuda.synchronize()
            free_before, _ = torch.cuda.mem_get_info(DEV)
            rc = lib.prism_b200_scan_static(n, got.data_ptr(), stream)
            assert rc == 0, _lib.last_error()
            torch.cuda.synchronize()
            free_after, _ = torch.cuda.mem_get_info(DEV)
            if call > 0:  # the first call may still trigger the runtime's own lazy set-up
                assert free_after >= free_before, "device memory was allocated during the call"
            assert torch.equal(got, want), f"call {call}: built-in scratch result differs from prism_b200_scan"
            assert np.array_equal(got.cpu().numpy().view(np.uint32), O.scan_cpu(src.cpu().numpy().view(np.uint32))), \
                f"call {call}: built-in scratch result differs from the oracle"
        assert _lib.last_error()[0] == 0


def test_static_scan_rejects_sizes_beyond_the_built_in_scratch():
    lib, _lib = _abi()
    x = torch.zeros(16, dtype=torch.int32, device=DEV)
    rc = lib.prism_b200_scan_static((1 << 28) + 1, x.data_ptr(), None)   # rejected before anything is launched
    assert rc == 6
    code, msg = _lib.last_error()
    assert code == 6 and "built-in scratch" in msg
    lib.prism_b200_clear_error()
    assert lib.prism_b200_scan_static(0, None, None) == 0
