// End-to-end timing of the three operators for a caller whose operands live in host memory,
// through the C ABI alone (no Python, no torch): pinned host arrays in, pinned host arrays out,
// every run = upload + kernels + download, as the reference harnesses do around their launches
// (evals/4090_scan/scan_harness.cuh:112-131, evals/h100_bench/main.cu:105-130).  Each result is
// spot-checked on the host.
//
//   host_e2e [gemm_size=8192] [sgemm_size=4096] [scan_log2n=28]
#include <chrono>
#include <cstdint>
#include <cstring>
#include <vector>

#include "common.h"

static uint16_t f32_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);   // round to nearest even (finite inputs only)
    return static_cast<uint16_t>(u >> 16);
}
static float bf16_to_f32(uint16_t h) {
    uint32_t u = static_cast<uint32_t>(h) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

template <typename F>
static double time_ms(int reps, F&& run) {
    run();   // warm-up
    EVAL_CUDA(cudaDeviceSynchronize());
    const auto t0 = std::chrono::high_resolution_clock::now();
    for (int r = 0; r < reps; ++r) run();
    EVAL_CUDA(cudaDeviceSynchronize());
    return std::chrono::duration<double, std::milli>(std::chrono::high_resolution_clock::now() - t0).count() / reps;
}

template <typename T>
static T* pinned(size_t count) {
    void* p = nullptr;
    EVAL_CUDA(cudaHostAlloc(&p, count * sizeof(T), cudaHostAllocDefault));
    return static_cast<T*>(p);
}

int main(int argc, char** argv) {
    const int gs = argc > 1 ? std::atoi(argv[1]) : 8192;
    const int ss = argc > 2 ? std::atoi(argv[2]) : 4096;
    const int lg = argc > 3 ? std::atoi(argv[3]) : 28;
    Lcg rng(2024);
    int bad = 0;

    if (gs > 0) {   // bf16 GEMM, C (N x M) = B * A^T
        const size_t S = gs;
        uint16_t *A = pinned<uint16_t>(S * S), *B = pinned<uint16_t>(S * S), *C = pinned<uint16_t>(S * S);
        for (size_t i = 0; i < S * S; ++i) {
            A[i] = f32_to_bf16(0.1f * rng.uniform_pm1());
            B[i] = f32_to_bf16(0.1f * rng.uniform_pm1());
        }
        prism_b200_host_plan* plan;
        eval_check(prism_b200_host_gemm_bf16_create(gs, gs, gs, 0, &plan), "host_gemm_bf16_create");
        const double ms = time_ms(5, [&] { eval_check(prism_b200_host_gemm_bf16_run(plan, A, B, C, nullptr), "host_gemm_bf16_run"); });
        for (size_t n : {size_t(0), S / 2 + 1, S - 1})
            for (size_t m : {size_t(0), S / 3, S - 1}) {
                double ref = 0;
                for (size_t k = 0; k < S; ++k) ref += double(bf16_to_f32(B[n * S + k])) * double(bf16_to_f32(A[m * S + k]));
                const double got = bf16_to_f32(C[n * S + m]);
                if (!(std::abs(got - ref) <= 1e-2 * std::abs(ref) + 1e-2)) { std::printf("bf16 GEMM mismatch at (%zu, %zu): %g vs %g\n", n, m, got, ref); ++bad; }
            }
        std::printf("host bf16 GEMM %d^3, %d blocks: %.3f ms per call, %.1f TFLOP/s end to end (%.0f MB up, %.0f MB down)\n", gs,
                    prism_b200_host_plan_blocks(plan), ms, 2.0 * S * S * S / ms / 1e9, 2 * S * S * 2 / 1e6, S * S * 2 / 1e6);
        prism_b200_host_plan_destroy(plan);
        cudaFreeHost(A); cudaFreeHost(B); cudaFreeHost(C);
    }

    if (ss > 0) {   // SGEMM, C = 1.5 A B + 0.5 C
        const size_t S = ss;
        float *A = pinned<float>(S * S), *B = pinned<float>(S * S), *C = pinned<float>(S * S);
        std::vector<float> C0(S * S);
        for (size_t i = 0; i < S * S; ++i) {
            A[i] = rng.uniform_pm1();
            B[i] = rng.uniform_pm1();
            C0[i] = C[i] = rng.uniform_pm1();
        }
        prism_b200_host_plan* plan;
        eval_check(prism_b200_host_sgemm_create(5, ss, ss, ss, 0, &plan), "host_sgemm_create");
        eval_check(prism_b200_host_sgemm_run(plan, 1.5f, A, B, 0.5f, C, nullptr), "host_sgemm_run");
        EVAL_CUDA(cudaDeviceSynchronize());
        for (size_t r : {size_t(0), S / 2, S - 1})
            for (size_t c : {size_t(1), S / 3, S - 1}) {
                double ref = 0;
                for (size_t k = 0; k < S; ++k) ref += double(A[r * S + k]) * double(B[k * S + c]);
                ref = 1.5 * ref + 0.5 * C0[r * S + c];
                if (!(std::abs(C[r * S + c] - ref) <= 1e-3)) { std::printf("SGEMM mismatch at (%zu, %zu): %g vs %g\n", r, c, C[r * S + c], ref); ++bad; }
            }
        const double ms = time_ms(5, [&] { eval_check(prism_b200_host_sgemm_run(plan, 1.5f, A, B, 0.5f, C, nullptr), "host_sgemm_run"); });
        std::printf("host SGEMM %d^3, %d blocks: %.3f ms per call, %.1f TFLOP/s end to end (%.0f MB up, %.0f MB down)\n", ss,
                    prism_b200_host_plan_blocks(plan), ms, 2.0 * S * S * S / ms / 1e9, 3 * S * S * 4 / 1e6, S * S * 4 / 1e6);
        prism_b200_host_plan_destroy(plan);
        cudaFreeHost(A); cudaFreeHost(B); cudaFreeHost(C);
    }

    if (lg > 0) {   // scan, in place
        const size_t n = size_t(1) << lg;
        uint32_t* x = pinned<uint32_t>(n);
        std::vector<uint32_t> in(n);
        for (size_t i = 0; i < n; ++i) x[i] = in[i] = rng.next() % 101;
        prism_b200_host_plan* plan;
        eval_check(prism_b200_host_scan_create(n, 0, &plan), "host_scan_create");
        eval_check(prism_b200_host_scan_run(plan, x, nullptr), "host_scan_run");
        EVAL_CUDA(cudaDeviceSynchronize());
        uint32_t acc = 0;
        for (size_t i = 0; i < n; ++i) {
            acc += in[i];
            if (x[i] != acc) { std::printf("scan mismatch at %zu: %u vs %u\n", i, x[i], acc); ++bad; break; }
        }
        const double ms = time_ms(3, [&] { eval_check(prism_b200_host_scan_run(plan, x, nullptr), "host_scan_run"); });
        std::printf("host scan 2^%d, %d blocks: %.3f ms per call, %.1f GB/s end to end at 8 B/element (%.0f MB up, %.0f MB down)\n", lg,
                    prism_b200_host_plan_blocks(plan), ms, 8.0 * n / ms / 1e6, n * 4 / 1e6, n * 4 / 1e6);
        prism_b200_host_plan_destroy(plan);
        cudaFreeHost(x);
    }
    std::printf(bad ? "FAILED\n" : "PASSED\n");
    return bad ? 1 : 0;
}
