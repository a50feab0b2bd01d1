// The reference's scan harness program (evals/4090_scan/main.cu), its main() and its harness header
// (evals/4090_scan/scan_harness.cuh) both UNMODIFIED and compiled from where they lie, running on
// libprism_b200.so instead of the reference's own kernel.  TEST INFRASTRUCTURE ONLY.
//
// How: the harness header reaches the kernel through two functions, scan_gpu::get_workspace_size and
// scan_gpu::launch_scan (scan_harness.cuh:112-131,152-160).  They are defined here over the C ABI, and
// the header is included once, bound to them (it carries `#pragma once`).  The reference's main.cu
// is then included with the token `scan_gpu` renamed, so that its own kernel and launch glue
// (main.cu:14-86) land in a namespace nothing refers to, its second inclusion of the header is a
// no-op, and what remains in effect is its main() (main.cu:94-126): the correctness sizes
// 16384 ... 64 Mi against scan_cpu, then the 64 Mi benchmark, printed in the program's own format.
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "prism_b200.h"

namespace scan_gpu {

size_t get_workspace_size(size_t n) {
    size_t bytes = 0;
    if (prism_b200_scan_workspace_size(n, &bytes) != PRISM_B200_OK) {
        char msg[256];
        prism_b200_last_error(nullptr, msg, sizeof msg);
        fprintf(stderr, "prism_b200: %s\n", msg);
        exit(1);
    }
    return bytes;
}

// Returns nullptr on a refused call, which the harness reports as "not yet implemented" and exits on.
uint32_t* launch_scan(size_t n, uint32_t* x, void* workspace) {
    return prism_b200_scan(n, x, workspace, /*stream=*/nullptr) == PRISM_B200_OK ? x : nullptr;
}

}  // namespace scan_gpu

#include "evals/4090_scan/scan_harness.cuh"   // run_tests, run_config, gen_random_data, scan_cpu: bound to the two functions above

#define scan_gpu reference_scan_gpu_not_called
#include "evals/4090_scan/main.cu"            // its kernel goes unused; its main() is the program
#undef scan_gpu
