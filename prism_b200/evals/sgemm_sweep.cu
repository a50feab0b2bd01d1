// SGEMM sweep against cuBLAS, the program behind the reference's SGEMM figure
// (evals/4090_sgemm/main.cu:13-230): correctness of kernels 1-5 against cuBLAS at 1024^3
// (absolute tolerance 0.01, runner.cu:105-117), then for every size the average of 10
// back-to-back launches.  Same output lines, so evals/plot_results.py:37-79 parses it.
//
//   sgemm_sweep [max_size]        sizes 256 ... max_size (default 8192), powers of two
#include <cublas_v2.h>

#include <cmath>
#include <vector>

#include "common.h"

static void cublas_fp32(cublasHandle_t h, int M, int N, int K, float alpha, const float* A, const float* B, float beta,
                        float* C) {
    // Row-major C = A * B is column-major C^T = B^T * A^T; pure FP32 compute.
    cublasGemmEx(h, CUBLAS_OP_N, CUBLAS_OP_N, N, M, K, &alpha, B, CUDA_R_32F, N, A, CUDA_R_32F, K, &beta, C, CUDA_R_32F,
                 N, CUBLAS_COMPUTE_32F_PEDANTIC, CUBLAS_GEMM_DEFAULT);
}

int main(int argc, char** argv) {
    const int max_size = argc > 1 ? std::atoi(argv[1]) : 8192;
    std::vector<int> sizes;
    for (int s = 256; s <= max_size; s *= 2) sizes.push_back(s);
    if (sizes.empty()) sizes.push_back(max_size);
    const int big = sizes.back();
    const float alpha = 0.5f, beta = 3.0f;  // the reference's values (main.cu:48)
    const int kernels[] = {1, 2, 3, 4, 5};
    const int repeat = 10;

    const size_t elems = static_cast<size_t>(big) * big;
    std::vector<float> hA(elems), hB(elems), hC(elems), out(elems), ref(elems);
    Lcg rng(2024);
    for (size_t i = 0; i < elems; ++i) { hA[i] = rng.uniform_pm1(); hB[i] = rng.uniform_pm1(); hC[i] = rng.uniform_pm1(); }
    float *dA, *dB, *dC, *dRef;
    EVAL_CUDA(cudaMalloc(&dA, elems * 4)); EVAL_CUDA(cudaMalloc(&dB, elems * 4));
    EVAL_CUDA(cudaMalloc(&dC, elems * 4)); EVAL_CUDA(cudaMalloc(&dRef, elems * 4));
    EVAL_CUDA(cudaMemcpy(dA, hA.data(), elems * 4, cudaMemcpyHostToDevice));
    EVAL_CUDA(cudaMemcpy(dB, hB.data(), elems * 4, cudaMemcpyHostToDevice));
    cublasHandle_t handle;
    if (cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS) { std::fprintf(stderr, "cublasCreate failed\n"); return 1; }

    std::printf("====================================\nCorrectness Check at size 1024\n====================================\n");
    {
        const int m = big < 1024 ? big : 1024;
        const size_t e = static_cast<size_t>(m) * m;
        EVAL_CUDA(cudaMemcpy(dRef, hC.data(), e * 4, cudaMemcpyHostToDevice));
        cublas_fp32(handle, m, m, m, alpha, dA, dB, beta, dRef);
        EVAL_CUDA(cudaMemcpy(ref.data(), dRef, e * 4, cudaMemcpyDeviceToHost));
        for (int k : kernels) {
            EVAL_CUDA(cudaMemcpy(dC, hC.data(), e * 4, cudaMemcpyHostToDevice));
            eval_check(prism_b200_sgemm(k, m, m, m, alpha, dA, dB, beta, dC, nullptr), "prism_b200_sgemm");
            EVAL_CUDA(cudaMemcpy(out.data(), dC, e * 4, cudaMemcpyDeviceToHost));
            bool ok = true;
            for (size_t i = 0; i < e && ok; ++i) {
                const double d = std::fabs(static_cast<double>(ref[i]) - out[i]);
                if (!(d <= 0.01)) {
                    std::printf("Divergence! Should %5.2f, Is %5.2f (Diff %5.2f) at %zu\n", ref[i], out[i], d, i);
                    ok = false;
                }
            }
            std::printf("[My Kernel %d] %s\n", k, ok ? "PASSED" : "FAILED");
            if (!ok) return 1;
        }
    }

    std::printf("\n====================================\nStarting Performance Sweep\n====================================\n");
    cudaEvent_t beg, end;
    EVAL_CUDA(cudaEventCreate(&beg)); EVAL_CUDA(cudaEventCreate(&end));
    for (int size : sizes) {
        const long m = size;
        const size_t e = static_cast<size_t>(m) * m;
        const double flops = 2.0 * m * m * m;
        std::printf("\n====================================\nSize: %ldx%ldx%ld\n====================================\n", m, m, m);
        float ms = 0.f;
        EVAL_CUDA(cudaMemcpy(dRef, hC.data(), e * 4, cudaMemcpyHostToDevice));
        std::printf("\n[cuBLAS FP32]\n");
        cublas_fp32(handle, size, size, size, alpha, dA, dB, beta, dRef);  // not timed: first call picks the algorithm
        EVAL_CUDA(cudaEventRecord(beg));
        for (int j = 0; j < repeat; ++j) cublas_fp32(handle, size, size, size, alpha, dA, dB, beta, dRef);
        EVAL_CUDA(cudaEventRecord(end)); EVAL_CUDA(cudaEventSynchronize(end)); EVAL_CUDA(cudaEventElapsedTime(&ms, beg, end));
        std::printf("Average elapsed time: (%7.6f) s, performance: (%7.1f) GFLOPS. size: (%ld).\n", ms / 1e3 / repeat,
                    repeat * flops * 1e-9 / (ms / 1e3), m);
        for (int k : kernels) {
            std::printf("\n[My Kernel %d]\n", k);
            EVAL_CUDA(cudaMemcpy(dC, hC.data(), e * 4, cudaMemcpyHostToDevice));
            EVAL_CUDA(cudaEventRecord(beg));
            for (int j = 0; j < repeat; ++j)
                eval_check(prism_b200_sgemm(k, size, size, size, alpha, dA, dB, beta, dC, nullptr), "prism_b200_sgemm");
            EVAL_CUDA(cudaEventRecord(end)); EVAL_CUDA(cudaEventSynchronize(end)); EVAL_CUDA(cudaEventElapsedTime(&ms, beg, end));
            std::printf("Average elapsed time: (%7.6f) s, performance: (%7.1f) GFLOPS. size: (%ld).\n", ms / 1e3 / repeat,
                        repeat * flops * 1e-9 / (ms / 1e3), m);
            std::fflush(stdout);
        }
    }
    cublasDestroy(handle);
    return 0;
}
