/*
 * CPU restatement in plain C of what the three kernel families compute.
 * TEST INFRASTRUCTURE ONLY: loaded by tests/ and by the CPU-baseline legs of
 * bench.py, never by the prism_b200 package.
 *
 * Build: gcc -O3 -march=native -fopenmp -shared -fPIC oracle_cpu.c -o liboracle_cpu.so
 * (oracle/build_ref.py does it).
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>

/* Inclusive prefix sum, running 32-bit accumulator.
 * Follows scan_cpu, evals/4090_scan/scan_harness.cuh:30-36. */
void oracle_scan_u32(size_t n, const uint32_t* x, uint32_t* out) {
    uint32_t acc = 0;
    for (size_t i = 0; i < n; ++i) {
        acc += x[i];
        out[i] = acc;
    }
}

/* C = alpha * A * B + beta * C, row-major fp32, k ascending, one fp32
 * accumulator per element: the arithmetic of generated/my_sgemm_kernel_1.cu:19-23
 * (the tiled kernels 2-5 keep the same k order per element).  Rows are shared
 * out over OpenMP threads; the i-k-j loop order only changes which element is
 * worked on, not the order of additions into any element. */
void oracle_sgemm_f32(int M, int N, int K, float alpha, const float* A, const float* B, float beta, float* C) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < M; ++i) {
        float acc[N > 0 ? N : 1];
        memset(acc, 0, sizeof(float) * (size_t)N);
        for (int k = 0; k < K; ++k) {
            const float a = A[(size_t)i * K + k];
            const float* b = B + (size_t)k * N;
            for (int j = 0; j < N; ++j) acc[j] += a * b[j];
        }
        float* c = C + (size_t)i * N;
        for (int j = 0; j < N; ++j) c[j] = alpha * acc[j] + beta * c[j];
    }
}

static inline float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u); /* round to nearest even */
    return (uint16_t)(u >> 16);
}

/* C[n * M + m] = bf16( sum_k A[m, k] * B[n, k] ), fp32 accumulation, A and B
 * K-contiguous bf16: the data contract of cutlass_my_h100_match_no_tail
 * (generated/cutlass_my_h100_match_no_tail.cu:313,347-354). */
void oracle_gemm_bf16(int M, int N, int K, const uint16_t* A, const uint16_t* B, uint16_t* C) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        for (int m = 0; m < M; ++m) {
            float acc = 0.f;
            const uint16_t* a = A + (size_t)m * K;
            const uint16_t* b = B + (size_t)n * K;
            for (int k = 0; k < K; ++k) acc += bf16_to_f32(a[k]) * bf16_to_f32(b[k]);
            C[(size_t)n * M + m] = f32_to_bf16(acc);
        }
    }
}
