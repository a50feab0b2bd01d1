// bf16 GEMM against cuBLAS at one size, the program behind the reference's bf16 figure
// (evals/h100_bench/main.cu:75-167): C = A * B^T, A and B K-major, C column-major; the result is
// compared with cuBLAS (absolute tolerance 0.1, main.cu:43-55), then both are timed as the average
// of 8 back-to-back launches.  Same two result lines, so evals/plot_results.py:18-34 parses them.
//
//   bf16_bench <size>             default 6144, as in the reference
#include <cublas_v2.h>
#include <cuda_bf16.h>

#include <cmath>
#include <random>
#include <vector>

#include "common.h"

int main(int argc, char** argv) {
    const long size = argc > 1 ? std::atol(argv[1]) : 2048 * 3;
    const long m = size, n = size, k = size;
    const size_t elems = static_cast<size_t>(size) * size;
    std::vector<__nv_bfloat16> hA(elems), hB(elems), hC(elems), hRef(elems);
    std::default_random_engine gen(69);  // the reference's seed
    std::normal_distribution<float> dist(0.f, 1.f);
    for (size_t i = 0; i < elems; ++i) hA[i] = __float2bfloat16(dist(gen));
    for (size_t i = 0; i < elems; ++i) hB[i] = __float2bfloat16(dist(gen));
    __nv_bfloat16 *dA, *dB, *dC, *dRef;
    EVAL_CUDA(cudaMalloc(&dA, elems * 2)); EVAL_CUDA(cudaMalloc(&dB, elems * 2));
    EVAL_CUDA(cudaMalloc(&dC, elems * 2)); EVAL_CUDA(cudaMalloc(&dRef, elems * 2));
    EVAL_CUDA(cudaMemcpy(dA, hA.data(), elems * 2, cudaMemcpyHostToDevice));
    EVAL_CUDA(cudaMemcpy(dB, hB.data(), elems * 2, cudaMemcpyHostToDevice));
    EVAL_CUDA(cudaMemset(dC, 0, elems * 2)); EVAL_CUDA(cudaMemset(dRef, 0, elems * 2));
    cublasHandle_t handle;
    if (cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS) { std::fprintf(stderr, "cublasCreate failed\n"); return 1; }
    // Column-major C (M x N) = A^T-stored-as-(K x M) transposed times B stored as (K x N).
    auto cublas_gemm = [&] {
        const float alpha = 1.f, beta = 0.f;
        cublasGemmEx(handle, CUBLAS_OP_T, CUBLAS_OP_N, m, n, k, &alpha, dA, CUDA_R_16BF, k, dB, CUDA_R_16BF, k, &beta, dRef,
                     CUDA_R_16BF, m, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    };
    auto ours = [&] {
        eval_check(prism_b200_gemm_bf16(m, n, k, reinterpret_cast<const uint16_t*>(dA), reinterpret_cast<const uint16_t*>(dB),
                                        reinterpret_cast<uint16_t*>(dC), nullptr), "prism_b200_gemm_bf16");
    };
    std::printf("Testing prism_b200_gemm_bf16\n");
    cublas_gemm();
    ours();
    EVAL_CUDA(cudaDeviceSynchronize());
    EVAL_CUDA(cudaMemcpy(hC.data(), dC, elems * 2, cudaMemcpyDeviceToHost));
    EVAL_CUDA(cudaMemcpy(hRef.data(), dRef, elems * 2, cudaMemcpyDeviceToHost));
    bool ok = true;
    for (size_t i = 0; i < elems && ok; ++i) {
        const float d = std::fabs(__bfloat162float(hRef[i]) - __bfloat162float(hC[i]));
        // the reference's absolute bound, scaled with sqrt(K) beyond the size it was written for (outputs grow like sqrt(K))
        const float tol = 0.1f * std::fmax(1.f, std::sqrt(static_cast<float>(k) / 8192.f)) + 0.008f * std::fabs(__bfloat162float(hRef[i]));
        if (!(d <= tol)) {
            std::printf("Divergence! Should %5.2f, Is %5.2f (Diff %5.2f) at %zu\n", __bfloat162float(hRef[i]),
                        __bfloat162float(hC[i]), d, i);
            ok = false;
        }
    }
    std::printf(ok ? "Passed correctness verification!\n" : "Failed to pass correctness verification against cuBLAS.\n");

    const int repeat = 8;
    cudaEvent_t beg, end;
    EVAL_CUDA(cudaEventCreate(&beg)); EVAL_CUDA(cudaEventCreate(&end));
    const double flops = 2.0 * m * n * k;
    float ms = 0.f;
    EVAL_CUDA(cudaEventRecord(beg));
    for (int j = 0; j < repeat; ++j) ours();
    EVAL_CUDA(cudaEventRecord(end)); EVAL_CUDA(cudaEventSynchronize(end)); EVAL_CUDA(cudaEventElapsedTime(&ms, beg, end));
    std::printf("Kernel:  Average elapsed time: (%7.6f) s, performance: (%7.1f) TFLOPS. size: (%ld).\n", ms / 1e3 / repeat,
                repeat * flops * 1e-9 / ms, m);
    EVAL_CUDA(cudaEventRecord(beg));
    for (int j = 0; j < repeat; ++j) cublas_gemm();
    EVAL_CUDA(cudaEventRecord(end)); EVAL_CUDA(cudaEventSynchronize(end)); EVAL_CUDA(cudaEventElapsedTime(&ms, beg, end));
    std::printf("cuBLAS:  Average elapsed time: (%7.6f) s, performance: (%7.1f) TFLOPS. size: (%ld).\n", ms / 1e3 / repeat,
                repeat * flops * 1e-9 / ms, m);
    cublasDestroy(handle);
    return ok ? 0 : 1;
}
