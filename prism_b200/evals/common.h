// Shared helpers of the evaluation programs: they drive libprism_b200 through its C
// ABI and print the line formats that the reference's plotting script parses
// (evals/plot_results.py:18-108), so that script works on their output unchanged.
#pragma once
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>

#include "../../include/prism_b200.h"

#define EVAL_CUDA(expr)                                                                           \
    do {                                                                                          \
        cudaError_t e_ = (expr);                                                                  \
        if (e_ != cudaSuccess) {                                                                  \
            std::fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); \
            std::exit(1);                                                                         \
        }                                                                                         \
    } while (0)

inline void eval_check(int status, const char* what) {
    if (status != PRISM_B200_OK) {
        char msg[256];
        prism_b200_last_error(nullptr, msg, sizeof msg);
        std::fprintf(stderr, "%s failed: status %d: %s\n", what, status, msg);
        std::exit(1);
    }
}

// A small deterministic generator (the reference seeds from the clock, evals/4090_sgemm/runner.cu:54-65).
struct Lcg {
    unsigned long long s;
    explicit Lcg(unsigned long long seed) : s(seed * 2862933555777941757ull + 3037000493ull) {}
    unsigned next() {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        return static_cast<unsigned>(s >> 33);
    }
    float uniform_pm1() { return static_cast<float>(next() & 0xFFFFFF) / 8388608.0f - 1.0f; }
};
