"""The device-side error path: a bounded wait that runs out is reported, nothing traps or hangs,
and the context keeps working.  The wait is made to run out by giving it 200 microseconds on a
barrier that nothing completes."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from oracle import cpu_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu


def test_bounded_wait_timeout_is_reported_and_context_survives(pb):
    from prism_b200 import _lib
    lib = _lib.load()
    pb.clear_error()
    with torch.cuda.device(0):
        assert lib.prism_b200_selftest_wait_timeout(200_000, None) == 0
        torch.cuda.synchronize()           # returns normally: the kernel gave up by itself
    code, msg = pb.last_error()
    assert code == 5 and "self-test" in msg, (code, msg)
    pb.clear_error()
    assert pb.last_error()[0] == 0
    # the same context still computes correctly
    x_np = O.scan_inputs(100003, seed=1, high=16)
    x = torch.from_numpy(x_np.view(np.int32).copy()).cuda()
    pb.scan_(x)
    torch.cuda.synchronize()
    assert np.array_equal(x.cpu().numpy().view(np.uint32), O.scan_cpu(x_np))
    assert pb.last_error()[0] == 0


def test_selftest_limit_is_validated(pb):
    from prism_b200 import _lib
    lib = _lib.load()
    assert lib.prism_b200_selftest_wait_timeout(0, None) == 1
    assert lib.prism_b200_selftest_wait_timeout(10**9, None) == 1
    pb.clear_error()
