// Stands in for evals/h100_bench/utils.cuh when the reference's bf16 benchmark program (evals/h100_bench/main.cu,
// UNMODIFIED) is compiled for a B200.  TEST INFRASTRUCTURE ONLY.
//
// The reference's utils.cuh holds the Hopper kernel's PTX wrappers (wgmma, sm_90a only: they do not assemble for
// sm_100a) and, at its end, the one function main.cu calls: prism_h100::runmyh100(M, N, K, A, B, C, DB)
// (utils.cuh:504-533).  oracle/build_ref.py puts this file, under the name utils.cuh, beside a symbolic link to the
// reference's main.cu, so that the program's `#include "utils.cuh"` (main.cu:32) finds it; everything else -- the
// inputs (normal(0, 1), seed 69), the cuBLAS comparison with its 0.1 bound, the timing of 8 back-to-back launches and
// the two result lines -- is the reference's own code, running on libprism_b200.so.
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "prism_b200.h"

namespace prism_h100 {

// DB is the reference's debug buffer, which its launcher never reads (utils.cuh:504-533).
inline void runmyh100(int M, int N, int K, bf16* A, bf16* B, bf16* C, int* DB) {
    (void)DB;
    if (prism_b200_gemm_bf16(M, N, K, reinterpret_cast<const uint16_t*>(A), reinterpret_cast<const uint16_t*>(B),
                             reinterpret_cast<uint16_t*>(C), /*stream=*/nullptr) != PRISM_B200_OK) {
        char msg[256];
        prism_b200_last_error(nullptr, msg, sizeof msg);
        fprintf(stderr, "prism_b200: %s\n", msg);
        exit(1);
    }
}

}  // namespace prism_h100
