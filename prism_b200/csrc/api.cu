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
// One status word per device index, pinned + mapped; the same addresses are valid on every device (UVA).
constexpr int kStatusWords = 64;
uint32_t* g_status = nullptr;
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
    cudaError_t e = cudaHostAlloc(&p, kStatusWords * sizeof(uint32_t), cudaHostAllocPortable | cudaHostAllocMapped);
    if (e != cudaSuccess) {
        g_status_failed = true;
        g_code = PRISM_B200_ERR_CUDA;
        snprintf(g_msg, sizeof(g_msg), "cudaHostAlloc(status word): %s", cudaGetErrorString(e));
        return nullptr;
    }
    memset(p, 0, kStatusWords * sizeof(uint32_t));
    g_status = static_cast<uint32_t*>(p);
    return g_status;
}

}  // namespace prism_b200

using namespace prism_b200;

// One warp waits, with the given limit, on a barrier phase that nothing completes, reports the
// timeout through the status word and returns: the path every kernel here takes when one of its
// bounded waits runs out, in its smallest form.
__global__ void selftest_wait_timeout_kernel(unsigned long long limit_ns) {
    __shared__ uint64_t bar;
    __shared__ uint32_t never;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        never = 0;
        fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (!mbar_wait_bounded(&bar, 0, &never, limit_ns)) raise_device_status(DEV_SELFTEST_TIMEOUT);
    }
}

extern "C" int prism_b200_selftest_wait_timeout(unsigned long long limit_ns, void* stream) {
    if (limit_ns == 0 || limit_ns > 10ull * 1000 * 1000)
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "selftest_wait_timeout: limit must be 1 ns .. 10 ms");
    if (int rc = bind_status_word()) return rc;
    selftest_wait_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns);
    PRISM_CUDA_TRY(cudaGetLastError());
    count_launch();
    return PRISM_B200_OK;
}

extern "C" int prism_b200_version(void) { return 100; }

extern "C" int prism_b200_last_error(int* code, char* msg, size_t len) {
    std::lock_guard<std::mutex> lk(g_mu);
    for (int d = 0; g_status && d < kStatusWords; ++d) {
        const uint32_t st = reinterpret_cast<volatile uint32_t*>(g_status)[d];
        if (st != DEV_OK) {
            g_code = PRISM_B200_ERR_DEVICE_TIMEOUT;
            const char* which = st == DEV_SCAN_LOOKBACK_TIMEOUT ? "scan look-back"
                              : st == DEV_SGEMM_PIPE_TIMEOUT    ? "sgemm smem pipeline"
                              : st == DEV_GEMM_PIPE_TIMEOUT     ? "bf16 gemm pipeline"
                              : st == DEV_SELFTEST_TIMEOUT      ? "self-test (as requested)"
                              : st == DEV_PEER_WAIT_TIMEOUT     ? "wait for the peers' blocks"
                                                                 : "unknown";
            snprintf(g_msg, sizeof(g_msg), "device %d: device-side wait ran out in %s (status 0x%08x)", d, which, st);
            break;
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
    for (int d = 0; g_status && d < kStatusWords; ++d) reinterpret_cast<volatile uint32_t*>(g_status)[d] = DEV_OK;
}

extern "C" unsigned long long prism_b200_launch_count(void) {
    return g_launches.load(std::memory_order_relaxed);
}
