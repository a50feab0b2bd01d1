// Exposes the reference's own CPU scan loop through a C symbol so that the
// oracle can be pinned against it.  TEST INFRASTRUCTURE ONLY.
//
// The reference source is compiled from where it lies: the include below is
// resolved with -I <reference root> (see oracle/build_ref.py); no reference
// source is copied into this repository.
#include <cstddef>
#include <cstdint>

// The harness header names these two launchers inside an inline function that
// this shim never calls; they only need to be declared.
namespace scan_gpu {
size_t get_workspace_size(size_t n);
uint32_t* launch_scan(size_t n, uint32_t* x, void* workspace);
}  // namespace scan_gpu

#include "evals/4090_scan/scan_harness.cuh"

extern "C" void ref_scan_cpu(size_t n, const uint32_t* x, uint32_t* out) { scan_cpu(n, x, out); }
