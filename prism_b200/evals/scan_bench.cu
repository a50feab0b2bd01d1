// Scan sweep against CUB, the program behind the reference's scan figure
// (evals/4090_scan/bench.cu:156-267): for n = 2^20 ... 2^30 both scans are checked element by
// element against a CPU loop and timed as the best single run inside a 500 ms window, host clock
// around launch + synchronise, input restored before every run (the reference re-uploads it from
// the host; here a device-to-device copy of the same data, untimed).  Same table as the reference,
// so evals/plot_results.py:82-108 parses it.
//
//   scan_bench [max_log2n]        default 30
#include <chrono>
#include <cstdint>
#include <cub/device/device_scan.cuh>
#include <limits>
#include <vector>

#include "common.h"

template <typename Reset, typename F>
static double best_ms(double window_ms, Reset&& reset, F&& f) {
    double best = std::numeric_limits<double>::infinity(), spent = 0.0;
    while (spent < window_ms) {
        reset();
        EVAL_CUDA(cudaDeviceSynchronize());
        const auto t0 = std::chrono::high_resolution_clock::now();
        f();
        EVAL_CUDA(cudaDeviceSynchronize());
        const double ms = std::chrono::duration<double, std::milli>(std::chrono::high_resolution_clock::now() - t0).count();
        spent += ms;
        if (ms < best) best = ms;
    }
    return best;
}

int main(int argc, char** argv) {
    const int max_log = argc > 1 ? std::atoi(argv[1]) : 30;
    std::printf("%-14s | %-10s %-14s | %-10s %-14s\n", "Size", "CUB (ms)", "CUB (GB/s)", "Ours (ms)", "Ours (GB/s)");
    std::printf("%-14s-+-%-10s-%-14s-+-%-10s-%-14s\n", "--------------", "----------", "--------------", "----------",
                "--------------");
    Lcg rng(0xCA7CAFE);
    for (int lg = 20; lg <= max_log; ++lg) {
        const size_t n = size_t(1) << lg;
        std::vector<uint32_t> in(n), expect(n), got(n);
        uint32_t acc = 0;
        for (size_t i = 0; i < n; ++i) {
            in[i] = rng.next() % 101;  // the reference's value range, uniform 0..100
            acc += in[i];
            expect[i] = acc;
        }
        const double bytes = static_cast<double>(n) * 4 * 2;
        uint32_t *d_src, *d_in, *d_out;
        EVAL_CUDA(cudaMalloc(&d_src, n * 4));
        EVAL_CUDA(cudaMalloc(&d_in, n * 4));
        EVAL_CUDA(cudaMalloc(&d_out, n * 4));
        EVAL_CUDA(cudaMemcpy(d_src, in.data(), n * 4, cudaMemcpyHostToDevice));

        // ---- CUB ----
        size_t cub_bytes = 0;
        cub::DeviceScan::InclusiveSum(nullptr, cub_bytes, d_in, d_out, n);
        void* d_cub;
        EVAL_CUDA(cudaMalloc(&d_cub, cub_bytes));
        // The scan is in place: every run starts from a fresh copy of the input (device to device, untimed).
        auto upload = [&] {
            EVAL_CUDA(cudaMemcpy(d_in, d_src, n * 4, cudaMemcpyDeviceToDevice));
            EVAL_CUDA(cudaDeviceSynchronize());
        };
        upload();
        cub::DeviceScan::InclusiveSum(d_cub, cub_bytes, d_in, d_out, n);
        EVAL_CUDA(cudaMemcpy(got.data(), d_out, n * 4, cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < n; ++i)
            if (got[i] != expect[i]) { std::printf("CUB mismatch at %zu: got %u expected %u\n", i, got[i], expect[i]); return 1; }
        const double cub_ms = best_ms(500.0, upload, [&] { cub::DeviceScan::InclusiveSum(d_cub, cub_bytes, d_in, d_out, n); });
        EVAL_CUDA(cudaFree(d_cub));
        EVAL_CUDA(cudaFree(d_out));

        // ---- ours (in place, like the reference's launch_scan) ----
        size_t ws_bytes = 0;
        eval_check(prism_b200_scan_workspace_size(n, &ws_bytes), "prism_b200_scan_workspace_size");
        void* d_ws;
        EVAL_CUDA(cudaMalloc(&d_ws, ws_bytes));
        upload();
        eval_check(prism_b200_scan(n, d_in, d_ws, nullptr), "prism_b200_scan");
        EVAL_CUDA(cudaMemcpy(got.data(), d_in, n * 4, cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < n; ++i)
            if (got[i] != expect[i]) { std::printf("Ours mismatch at %zu: got %u expected %u\n", i, got[i], expect[i]); return 1; }
        const double our_ms = best_ms(500.0, upload, [&] { eval_check(prism_b200_scan(n, d_in, d_ws, nullptr), "prism_b200_scan"); });
        EVAL_CUDA(cudaFree(d_ws));
        EVAL_CUDA(cudaFree(d_in));
        EVAL_CUDA(cudaFree(d_src));

        std::printf("%-14zu | %-10.3f %-14.2f | %-10.3f %-14.2f\n", n, cub_ms, bytes / cub_ms / 1e6, our_ms,
                    bytes / our_ms / 1e6);
        std::fflush(stdout);
    }
    return 0;
}
