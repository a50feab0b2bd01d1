"""Writes tests/golden/sgemm_ref_gpu.npz: outputs of the reference's own SGEMM kernels 1-5
(generated/my_sgemm_kernel_*.cu and sgemm_shared_mem_block.cu, recompiled for sm_100 with the
harness launch geometry by oracle/build_ref.py) on one seeded 128^3 problem.  Needs a GPU and
oracle/_ref/libprism_ref.so:

    python oracle/build_ref.py && python tests/golden/make_golden_gpu.py [out.npz]
"""
import ctypes
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import cpu_oracle as O  # noqa: E402


def main():
    out_path = Path(sys.argv[1]) if len(sys.argv) > 1 else ROOT / "tests" / "golden" / "sgemm_ref_gpu.npz"
    lib = ctypes.CDLL(str(ROOT / "oracle" / "_ref" / "libprism_ref.so"))
    lib.ref_sgemm.argtypes = [ctypes.c_int] * 4 + [ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float,
                                                   ctypes.c_void_p]
    M = N = K = 128
    alpha, beta = 1.5, 0.5
    A, B, C = O.sgemm_inputs(M, N, K, seed=128)
    a, b = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    out = {"A": A, "B": B, "C": C, "alpha": np.float32(alpha), "beta": np.float32(beta)}
    for k in (1, 2, 3, 4, 5):
        c = torch.from_numpy(C).cuda()
        torch.cuda.synchronize()
        assert lib.ref_sgemm(k, M, N, K, alpha, a.data_ptr(), b.data_ptr(), beta, c.data_ptr()) == 0
        torch.cuda.synchronize()
        out[f"out_k{k}"] = c.cpu().numpy()
    np.savez_compressed(out_path, **out)
    print("wrote", out_path)


if __name__ == "__main__":
    main()
