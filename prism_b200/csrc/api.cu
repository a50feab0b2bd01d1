// Library-level entry points: version, sticky error state, launch counter and
// the pinned status word that kernels use to report a wait that ran out.
#include "common.cuh"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

namespace prism_b200 {

namespace {
std::mutex g_mu;
int g_code = 0;
char g_msg[256] = "";
std::atomic<unsigned long long> g_launches{0};
uint32_t* g_status = nullptr;  // pinned + mapped; the same address is valid on every device (UVA)
bool g_status_failed = false;
}  // namespace

int set_error(int code, const char* fmt, ...) {
    std::lock_guard<std::mutex> lk(g_mu);
    g_code = code;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_msg, sizeof(g_msg), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_failed(cudaError_t e, const char* what) {
    return set_error(PRISM_B200_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

void count_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

uint32_t* device_status_word() {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_status || g_status_failed) return g_status;
    void* p = nullptr;
    cudaError_t e = cudaHostAlloc(&p, 64, cudaHostAllocPortable | cudaHostAllocMapped);
    if (e != cudaSuccess) {
        g_status_failed = true;
        g_code = PRISM_B200_ERR_CUDA;
        snprintf(g_msg, sizeof(g_msg), "cudaHostAlloc(status word): %s", cudaGetErrorString(e));
        return nullptr;
    }
    memset(p, 0, 64);
    g_status = static_cast<uint32_t*>(p);
    return g_status;
}

}  // namespace prism_b200

using namespace prism_b200;

extern "C" int prism_b200_version(void) { return 100; }

extern "C" int prism_b200_last_error(int* code, char* msg, size_t len) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_status) {
        uint32_t dev = *reinterpret_cast<volatile uint32_t*>(g_status);
        if (dev != DEV_OK) {
            g_code = PRISM_B200_ERR_DEVICE_TIMEOUT;
            const char* which = dev == DEV_SCAN_LOOKBACK_TIMEOUT ? "scan look-back"
                              : dev == DEV_SGEMM_PIPE_TIMEOUT    ? "sgemm smem pipeline"
                              : dev == DEV_GEMM_PIPE_TIMEOUT     ? "bf16 gemm pipeline"
                                                                  : "unknown";
            snprintf(g_msg, sizeof(g_msg), "device-side wait ran out in %s (status 0x%08x)", which, dev);
        }
    }
    if (code) *code = g_code;
    if (msg && len) {
        strncpy(msg, g_msg, len - 1);
        msg[len - 1] = '\0';
    }
    return g_code;
}

extern "C" void prism_b200_clear_error(void) {
    std::lock_guard<std::mutex> lk(g_mu);
    g_code = 0;
    g_msg[0] = '\0';
    if (g_status) *reinterpret_cast<volatile uint32_t*>(g_status) = DEV_OK;
}

extern "C" unsigned long long prism_b200_launch_count(void) {
    return g_launches.load(std::memory_order_relaxed);
}
