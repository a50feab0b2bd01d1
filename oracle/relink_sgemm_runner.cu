// TEST INFRASTRUCTURE ONLY.  Stand-in for the reference's evals/4090_sgemm/runner.cu when its
// sweep program (evals/4090_sgemm/main.cu) is compiled, unmodified and from where it lies, against
// this library: the functions that program calls through runner.cuh, written afresh, with
// `run_my_kernel` (runner.cu:245-267) forwarding to prism_b200_sgemm.  Built by build_ref.py into
// oracle/_ref/relink_sgemm_sweep; shows that the reference harness needs no change beyond the link line.
#include <runner.cuh>

#include <cmath>
#include <cstdio>
#include <cstdlib>

#include "prism_b200.h"

void(cudaCheck)(cudaError_t error, const char* file, int line) {
    if (error == cudaSuccess) return;
    std::fprintf(stderr, "CUDA error at %s:%d: %s\n", file, line, cudaGetErrorString(error));
    std::exit(EXIT_FAILURE);
}

void CudaDeviceInfo() {
    int dev = 0;
    cudaDeviceProp p{};
    if (cudaGetDevice(&dev) == cudaSuccess && cudaGetDeviceProperties(&p, dev) == cudaSuccess)
        std::printf("device %d: %s, %d SMs, %.1f GiB\n", dev, p.name, p.multiProcessorCount, p.totalGlobalMem / 1073741824.0);
}

// Values with two decimals in (-5, 5), as the reference draws them; the generator is ours (a 64-bit LCG).
void randomize_matrix(float* mat, int N) {
    static unsigned long long state = 0x9E3779B97F4A7C15ull;
    auto next = [&]() {
        state = state * 6364136223846793005ull + 1442695040888963407ull;
        return static_cast<unsigned>(state >> 33);
    };
    for (int i = 0; i < N; ++i) {
        float v = static_cast<float>(next() % 5) + 0.01f * static_cast<float>(next() % 5);
        mat[i] = (next() & 1u) ? -v : v;
    }
}

void range_init_matrix(float* mat, int N) {
    for (int i = 0; i < N; ++i) mat[i] = static_cast<float>(i);
}

void zero_init_matrix(float* mat, int N) {
    for (int i = 0; i < N; ++i) mat[i] = 0.f;
}

void copy_matrix(const float* src, float* dest, int N) {
    for (int i = 0; i < N; ++i) dest[i] = src[i];
}

void print_matrix(const float* A, int M, int N, std::ofstream& fs) {
    for (int r = 0; r < M; ++r) {
        for (int c = 0; c < N; ++c) fs << A[static_cast<size_t>(r) * N + c] << (c + 1 < N ? ", " : "\n");
    }
}

// Same acceptance rule as the reference (runner.cu:105-117): absolute difference at most 0.01, NaN fails.
bool verify_matrix(float* ref, float* out, int N) {
    for (int i = 0; i < N; ++i) {
        const double d = std::fabs(static_cast<double>(ref[i]) - static_cast<double>(out[i]));
        if (!(d <= 0.01)) {
            std::printf("Divergence! Should %5.2f, Is %5.2f (Diff %5.2f) at %d\n", ref[i], out[i], d, i);
            return false;
        }
    }
    return true;
}

float get_current_sec() {
    timeval tv{};
    gettimeofday(&tv, nullptr);
    return static_cast<float>(tv.tv_sec) + 1e-6f * static_cast<float>(tv.tv_usec);
}

float cpu_elapsed_time(float& beg, float& end) { return end - beg; }

// Kernel 0 is the cuBLAS fp32 product of row-major operands: C^T = B^T * A^T in cuBLAS's column-major terms.
void run_kernel(int kernel_num, int m, int n, int k, float alpha, float* A, float* B, float beta, float* C,
                cublasHandle_t handle) {
    if (kernel_num != 0) {
        std::fprintf(stderr, "run_kernel: only kernel 0 (cuBLAS) is provided by this stand-in\n");
        std::exit(EXIT_FAILURE);
    }
    cublasSetMathMode(handle, CUBLAS_PEDANTIC_MATH);  // no TF32
    const cublasStatus_t st = cublasSgemm(handle, CUBLAS_OP_N, CUBLAS_OP_N, n, m, k, &alpha, B, n, A, k, &beta, C, n);
    if (st != CUBLAS_STATUS_SUCCESS) {
        std::fprintf(stderr, "cublasSgemm failed: %d\n", static_cast<int>(st));
        std::exit(EXIT_FAILURE);
    }
}

void run_my_kernel(int my_kernel_num, int m, int n, int k, float alpha, float* A, float* B, float beta, float* C) {
    if (prism_b200_sgemm(my_kernel_num, m, n, k, alpha, A, B, beta, C, nullptr) != PRISM_B200_OK) {
        char msg[256];
        int code = 0;
        prism_b200_last_error(&code, msg, sizeof msg);
        std::fprintf(stderr, "prism_b200_sgemm(kernel %d) failed: %d %s\n", my_kernel_num, code, msg);
        std::exit(EXIT_FAILURE);
    }
}
