// Shared host/device plumbing for the prism_b200 kernels: status codes, the
// sticky error state, the pinned device-visible status word and small PTX helpers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

#include <mutex>

#include "../../include/prism_b200.h"

namespace prism_b200 {

// ---- host-side error state (api.cu) ---------------------------------------
int  set_error(int code, const char* fmt, ...);
int  cuda_failed(cudaError_t e, const char* what);
void count_launch(unsigned n = 1);

// Device-visible status words in pinned, mapped host memory, one per device index (64).
// Kernels write a non-zero code into their device's word when a bounded wait gives up;
// the host reads them without a CUDA call.  Returns the first word's address, or nullptr
// (and sets the error state) if the buffer cannot be set up.
uint32_t* device_status_word();

// Codes written into the status word by kernels.
enum : uint32_t {
    DEV_OK = 0,
    DEV_SCAN_LOOKBACK_TIMEOUT = 0x5CA10001u,
    DEV_SGEMM_PIPE_TIMEOUT    = 0x56E30001u,  // reserved: the SGEMM kernels have no waits that can run out
    DEV_GEMM_PIPE_TIMEOUT     = 0xB16E0001u,
    DEV_SELFTEST_TIMEOUT      = 0x5E1F0001u,
    DEV_PEER_WAIT_TIMEOUT     = 0x9EE20001u,
};

#define PRISM_CUDA_TRY(expr)                                            \
    do {                                                                \
        cudaError_t _e = (expr);                                        \
        if (_e != cudaSuccess) return ::prism_b200::cuda_failed(_e, #expr); \
    } while (0)

// ---- device helpers -----------------------------------------------------------
#ifdef __CUDACC__

// Each translation unit keeps its own device-side copy of the status word's
// address (no relocatable device code needed).  bind_status_word() fills it in
// once per device; the first call on a device does a small synchronous copy, so
// it should come before any stream capture.
static __device__ uint32_t* d_status_word;

static inline int bind_status_word() {
    static bool bound[64] = {};
    static std::mutex mu;   // entry points may be called from several host threads
    std::lock_guard<std::mutex> lk(mu);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_failed(e, "cudaGetDevice");
    if (dev >= 0 && dev < 64 && bound[dev]) return PRISM_B200_OK;
    uint32_t* p = device_status_word();
    if (!p) return PRISM_B200_ERR_CUDA;
    if (dev >= 0 && dev < 64) p += dev;   // this device's own word
    e = cudaMemcpyToSymbol(d_status_word, &p, sizeof(p));
    if (e != cudaSuccess) return cuda_failed(e, "cudaMemcpyToSymbol(status word)");
    if (dev >= 0 && dev < 64) bound[dev] = true;
    return PRISM_B200_OK;
}

__device__ __forceinline__ void raise_device_status(uint32_t code) {
    if (d_status_word) *reinterpret_cast<volatile uint32_t*>(d_status_word) = code;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Longest time any single wait inside a kernel may take before the kernel gives
// up, raises its status code and unwinds.  Real waits last microseconds.
constexpr unsigned long long kWaitLimitNs = 1000ull * 1000ull * 1000ull;

// Bounded wait on an mbarrier phase.  Returns false when the time limit passed
// or when *abort_flag (shared memory) became non-zero; the caller then unwinds
// instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  volatile uint32_t* abort_flag,
                                                  unsigned long long limit_ns = kWaitLimitNs) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    for (uint32_t i = 1;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 0u) {
            if (*abort_flag) return false;
            if (global_timer_ns() - t0 > limit_ns) return false;
        }
    }
}

// The same wait for a role that can afford to react late: sleeps between probes, so that a warp
// that waits for tens of microseconds does not spend issue slots and power on polling.
__device__ __forceinline__ bool mbar_wait_bounded_sleepy(uint64_t* bar, uint32_t parity,
                                                         volatile uint32_t* abort_flag, unsigned sleep_ns,
                                                         unsigned long long limit_ns = kWaitLimitNs) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    for (uint32_t i = 1;; ++i) {
        __nanosleep(sleep_ns);
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 15u) == 0u) {
            if (*abort_flag) return false;
            if (global_timer_ns() - t0 > limit_ns) return false;
        }
    }
}

__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

#endif  // __CUDACC__

}  // namespace prism_b200
