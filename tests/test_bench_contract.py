"""bench.py's reference arm runs on CPU and must print one JSON line with the contract's keys."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("workload", ["gemm_bf16", "scan"])
def test_reference_arm_prints_one_json_line(workload):
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                        "--workload", workload], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["value"] > 0 and d["higher_is_better"] is True
    assert d["cpu_baseline"]["kind"] in ("port", "reference") and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in d["config"]


def test_own_arm_fails_loudly_without_a_gpu():
    """There is no CPU path: without a CUDA device the kernel arm must exit non-zero and say why."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--steps", "1", "--warmup", "1"], capture_output=True,
                       text=True, timeout=300)
    assert r.returncode != 0
    assert "no CPU path" in r.stdout


def test_reference_arm_uses_every_core_under_a_launcher_that_exports_one_thread():
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the CPU arm must undo that before BLAS loads,
    and must carry the same `config` as the GPU arm (M, N, K, sharding for the number of GPUs)."""
    import os
    env = dict(os.environ, OMP_NUM_THREADS="1", RANK="0", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                        "--warmup", "0"], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    d = json.loads(r.stdout.strip().splitlines()[-1])
    want = len(os.sched_getaffinity(0))
    assert d["cpu_baseline"]["cores"] == want, d["cpu_baseline"]
    assert d["config"]["M"] == d["config"]["N"] == d["config"]["K"] == 8192 and d["config"]["rows_per_gpu"] == 4096
    # a rank other than 0 prints nothing and exits 0
    env["RANK"] = "1"
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                        "--warmup", "0"], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""
