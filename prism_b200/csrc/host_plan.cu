// Host-buffer plans: the three operators for callers whose operands live in host memory,
// as the reference harnesses' do (they cudaMemcpy around every launch:
// evals/4090_scan/scan_harness.cuh:112-131, evals/h100_bench/main.cu:105-130).
//
// The host link is the bottleneck of each of them (the kernels take about a tenth of the
// copy time), so a plan owns device staging buffers and three streams, cuts a call into
// blocks that are contiguous on both sides and overlaps the upload of block j+1, the
// kernel on block j and the download of block j-1; uploads and downloads use the two
// directions of the link at once.
//   bf16 GEMM: A whole, then B in blocks of rows; rows of B are columns of the
//              column-major C, i.e. contiguous row blocks of the N x M result.
//   SGEMM:     B whole, then A and C in blocks of rows of M.
//   scan:      blocks of the array; each block starts from the last element of the block
//              before it, which stays on the device.
// A run is ordered after the work already queued on the caller's stream, and the caller's
// stream waits for it; nothing here blocks the host.
#include "common.cuh"

#include <vector>

using namespace prism_b200;

namespace {
enum Kind { kGemmBF16 = 1, kSgemm = 2, kScan = 3 };
constexpr uint32_t kMagic = 0x504C414Eu;  // "PLAN"
constexpr size_t kMaxBlocks = 256;
}  // namespace

struct prism_b200_host_plan {
    uint32_t magic = kMagic;
    int kind = 0;
    int device = 0;
    int M = 0, N = 0, K = 0, kernel_id = 0;
    size_t n = 0;
    void *a = nullptr, *b = nullptr, *c = nullptr;   // device staging (scan: a = the array, b = workspace, c = carry word)
    cudaStream_t lane[3] = {};                        // upload, kernel, download
    cudaEvent_t begin = nullptr, done[3] = {};
    std::vector<cudaEvent_t> uploaded, computed;
    std::vector<std::pair<size_t, size_t>> blocks;   // [lo, hi) in rows (GEMMs) or elements (scan)
};

namespace {

// Cuts [0, n) into blocks of `block` (a multiple of `quantum`).  With `taper` the last block is cut again and again
// in halves down to `quantum`: what remains to be done after the last byte has gone up is the last block's kernel
// and download, so the last block should be small, while the earlier ones stay large enough to keep the kernel
// efficient (1024, ..., 1024, 512, 256, 256 for n = 8192, block = 1024, quantum = 256).
void cut(std::vector<std::pair<size_t, size_t>>& out, size_t n, size_t block, size_t quantum, bool taper = false) {
    out.clear();
    if (n == 0) return;
    if (n % quantum != 0 || n <= block) {
        out.emplace_back(0, n);
        return;
    }
    block = block / quantum * quantum;
    if (block < quantum) block = quantum;
    if ((n + block - 1) / block > kMaxBlocks) block = ((n + kMaxBlocks - 1) / kMaxBlocks + quantum - 1) / quantum * quantum;
    for (size_t lo = 0; lo < n; lo += block) out.emplace_back(lo, lo + block < n ? lo + block : n);
    while (taper && out.size() < kMaxBlocks) {
        const size_t lo = out.back().first, hi = out.back().second;
        const size_t half = (hi - lo) / 2 / quantum * quantum;
        if (half < quantum || hi - lo - half < quantum) break;
        out.back().second = lo + half;
        out.emplace_back(lo + half, hi);
    }
}

void destroy(prism_b200_host_plan* p) {
    if (!p) return;
    cudaFree(p->a);
    cudaFree(p->b);
    cudaFree(p->c);
    for (auto& s : p->lane)
        if (s) cudaStreamDestroy(s);
    if (p->begin) cudaEventDestroy(p->begin);
    for (auto& e : p->done)
        if (e) cudaEventDestroy(e);
    for (auto e : p->uploaded) cudaEventDestroy(e);
    for (auto e : p->computed) cudaEventDestroy(e);
    p->magic = 0;
    delete p;
}

int finish_create(prism_b200_host_plan* p, size_t bytes_a, size_t bytes_b, size_t bytes_c, prism_b200_host_plan** out) {
    cudaError_t e = cudaGetDevice(&p->device);
    if (e == cudaSuccess && bytes_a) e = cudaMalloc(&p->a, bytes_a);
    if (e == cudaSuccess && bytes_b) e = cudaMalloc(&p->b, bytes_b);
    if (e == cudaSuccess && bytes_c) e = cudaMalloc(&p->c, bytes_c);
    for (auto& s : p->lane)
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->begin, cudaEventDisableTiming);
    for (auto& d : p->done)
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&d, cudaEventDisableTiming);
    for (size_t j = 0; j < p->blocks.size() && e == cudaSuccess; ++j) {
        cudaEvent_t u = nullptr, k = nullptr;
        e = cudaEventCreateWithFlags(&u, cudaEventDisableTiming);
        if (e == cudaSuccess) p->uploaded.push_back(u);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&k, cudaEventDisableTiming);
        if (e == cudaSuccess) p->computed.push_back(k);
    }
    if (e != cudaSuccess) {
        destroy(p);
        return cuda_failed(e, "host plan set-up");
    }
    *out = p;
    return PRISM_B200_OK;
}

int check_plan(const prism_b200_host_plan* p, int kind, const char* what) {
    if (!p || p->magic != kMagic || p->kind != kind)
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "%s: not a plan of this kind", what);
    int dev = -1;
    PRISM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev != p->device)
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "%s: plan was made on device %d, current device is %d", what,
                         p->device, dev);
    return PRISM_B200_OK;
}

int begin_run(prism_b200_host_plan* p, cudaStream_t caller) {
    PRISM_CUDA_TRY(cudaEventRecord(p->begin, caller));
    for (auto s : p->lane) PRISM_CUDA_TRY(cudaStreamWaitEvent(s, p->begin, 0));
    return PRISM_B200_OK;
}

int end_run(prism_b200_host_plan* p, cudaStream_t caller) {
    for (int i = 0; i < 3; ++i) {
        PRISM_CUDA_TRY(cudaEventRecord(p->done[i], p->lane[i]));
        PRISM_CUDA_TRY(cudaStreamWaitEvent(caller, p->done[i], 0));
    }
    return PRISM_B200_OK;
}

// A kernel entry point refused mid-run: the copies already queued still run, so the caller's stream
// is tied to the lanes as at the end of a normal run before the error goes back (the error state
// keeps the kernel's message).
int abandon_run(prism_b200_host_plan* p, cudaStream_t caller, int rc) {
    for (int i = 0; i < 3; ++i)
        if (cudaEventRecord(p->done[i], p->lane[i]) == cudaSuccess) cudaStreamWaitEvent(caller, p->done[i], 0);
    return rc;
}

// Inside a run: a CUDA call that fails after copies have been queued goes through abandon_run, so that the
// caller's stream still waits for what is already in flight on the plan's lanes.
#define PRISM_RUN_TRY(expr)                                                              \
    do {                                                                                 \
        cudaError_t _e = (expr);                                                         \
        if (_e != cudaSuccess) return abandon_run(p, caller, ::prism_b200::cuda_failed(_e, #expr)); \
    } while (0)

}  // namespace

extern "C" int prism_b200_host_gemm_bf16_create(int M, int N, int K, int block_rows, prism_b200_host_plan** plan) {
    if (!plan) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "host_gemm_bf16_create: null plan pointer");
    *plan = nullptr;
    if (M <= 0 || N <= 0 || K <= 0 || block_rows < 0)
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "host_gemm_bf16_create: dimensions must be positive");
    auto* p = new prism_b200_host_plan;
    p->kind = kGemmBF16;
    p->M = M; p->N = N; p->K = K;
    cut(p->blocks, static_cast<size_t>(N), block_rows ? block_rows : 1024, 256, /*taper=*/block_rows == 0);
    return finish_create(p, static_cast<size_t>(M) * K * 2, static_cast<size_t>(N) * K * 2, static_cast<size_t>(N) * M * 2, plan);
}

extern "C" int prism_b200_host_gemm_bf16_run(prism_b200_host_plan* p, const uint16_t* A_host, const uint16_t* B_host,
                                             uint16_t* C_host, void* stream) {
    if (int rc = check_plan(p, kGemmBF16, "host_gemm_bf16_run")) return rc;
    if (!A_host || !B_host || !C_host) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "host_gemm_bf16_run: null pointer");
    cudaStream_t caller = static_cast<cudaStream_t>(stream);
    if (int rc = begin_run(p, caller)) return rc;
    const size_t row_b = static_cast<size_t>(p->K) * 2, row_c = static_cast<size_t>(p->M) * 2;
    PRISM_RUN_TRY(cudaMemcpyAsync(p->a, A_host, static_cast<size_t>(p->M) * row_b, cudaMemcpyHostToDevice, p->lane[0]));
    for (size_t j = 0; j < p->blocks.size(); ++j) {
        const size_t lo = p->blocks[j].first, rows = p->blocks[j].second - lo;
        char* b_dev = static_cast<char*>(p->b) + lo * row_b;
        char* c_dev = static_cast<char*>(p->c) + lo * row_c;
        PRISM_RUN_TRY(cudaMemcpyAsync(b_dev, reinterpret_cast<const char*>(B_host) + lo * row_b, rows * row_b,
                                       cudaMemcpyHostToDevice, p->lane[0]));
        PRISM_RUN_TRY(cudaEventRecord(p->uploaded[j], p->lane[0]));
        PRISM_RUN_TRY(cudaStreamWaitEvent(p->lane[1], p->uploaded[j], 0));
        if (int rc = prism_b200_gemm_bf16(p->M, static_cast<int>(rows), p->K, static_cast<const uint16_t*>(p->a),
                                          reinterpret_cast<const uint16_t*>(b_dev), reinterpret_cast<uint16_t*>(c_dev),
                                          p->lane[1]))
            return abandon_run(p, caller, rc);
        PRISM_RUN_TRY(cudaEventRecord(p->computed[j], p->lane[1]));
        PRISM_RUN_TRY(cudaStreamWaitEvent(p->lane[2], p->computed[j], 0));
        PRISM_RUN_TRY(cudaMemcpyAsync(reinterpret_cast<char*>(C_host) + lo * row_c, c_dev, rows * row_c, cudaMemcpyDeviceToHost,
                                       p->lane[2]));
    }
    return end_run(p, caller);
}

extern "C" int prism_b200_host_sgemm_create(int kernel_id, int M, int N, int K, int block_rows,
                                            prism_b200_host_plan** plan) {
    if (!plan) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "host_sgemm_create: null plan pointer");
    *plan = nullptr;
    if (M <= 0 || N <= 0 || K <= 0 || block_rows < 0 || kernel_id < 1 || kernel_id > 6)
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "host_sgemm_create: bad dimensions or kernel id");
    auto* p = new prism_b200_host_plan;
    p->kind = kSgemm;
    p->M = M; p->N = N; p->K = K; p->kernel_id = kernel_id;
    // Default: sixteen blocks (4096^3 end to end on a B200: 4.40 ms against 4.52 with blocks of 1024 rows and 4.60 with 128).
    const int default_rows = ((M / 16 + 127) / 128) * 128;
    cut(p->blocks, static_cast<size_t>(M), block_rows ? block_rows : (default_rows > 128 ? default_rows : 128), 128,
        /*taper=*/block_rows == 0);
    return finish_create(p, static_cast<size_t>(M) * K * 4, static_cast<size_t>(K) * N * 4, static_cast<size_t>(M) * N * 4, plan);
}

extern "C" int prism_b200_host_sgemm_run(prism_b200_host_plan* p, float alpha, const float* A_host, const float* B_host,
                                         float beta, float* C_host, void* stream) {
    if (int rc = check_plan(p, kSgemm, "host_sgemm_run")) return rc;
    if (!A_host || !B_host || !C_host) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "host_sgemm_run: null pointer");
    cudaStream_t caller = static_cast<cudaStream_t>(stream);
    if (int rc = begin_run(p, caller)) return rc;
    const size_t K = p->K, N = p->N;
    PRISM_RUN_TRY(cudaMemcpyAsync(p->b, B_host, K * N * 4, cudaMemcpyHostToDevice, p->lane[0]));
    for (size_t j = 0; j < p->blocks.size(); ++j) {
        const size_t lo = p->blocks[j].first, rows = p->blocks[j].second - lo;
        float* a_dev = static_cast<float*>(p->a) + lo * K;
        float* c_dev = static_cast<float*>(p->c) + lo * N;
        PRISM_RUN_TRY(cudaMemcpyAsync(a_dev, A_host + lo * K, rows * K * 4, cudaMemcpyHostToDevice, p->lane[0]));
        PRISM_RUN_TRY(cudaMemcpyAsync(c_dev, C_host + lo * N, rows * N * 4, cudaMemcpyHostToDevice, p->lane[0]));
        PRISM_RUN_TRY(cudaEventRecord(p->uploaded[j], p->lane[0]));
        PRISM_RUN_TRY(cudaStreamWaitEvent(p->lane[1], p->uploaded[j], 0));
        if (int rc = prism_b200_sgemm(p->kernel_id, static_cast<int>(rows), p->N, p->K, alpha, a_dev,
                                      static_cast<const float*>(p->b), beta, c_dev, p->lane[1]))
            return abandon_run(p, caller, rc);
        PRISM_RUN_TRY(cudaEventRecord(p->computed[j], p->lane[1]));
        PRISM_RUN_TRY(cudaStreamWaitEvent(p->lane[2], p->computed[j], 0));
        PRISM_RUN_TRY(cudaMemcpyAsync(C_host + lo * N, c_dev, rows * N * 4, cudaMemcpyDeviceToHost, p->lane[2]));
    }
    return end_run(p, caller);
}

extern "C" int prism_b200_host_scan_create(size_t n, size_t block_elems, prism_b200_host_plan** plan) {
    if (!plan) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "host_scan_create: null plan pointer");
    *plan = nullptr;
    if (n >= (1ull << 32)) return set_error(PRISM_B200_ERR_TOO_LARGE, "host_scan_create: n must be below 2^32");
    auto* p = new prism_b200_host_plan;
    p->kind = kScan;
    p->n = n;
    if (block_elems == 0) block_elems = n / 16 > (size_t(1) << 22) ? n / 16 : (size_t(1) << 22);
    cut(p->blocks, n, block_elems, 4);   // block starts stay 16-byte aligned
    size_t longest = 0, ws = 0;
    for (auto& b : p->blocks) longest = b.second - b.first > longest ? b.second - b.first : longest;
    if (int rc = prism_b200_scan_workspace_size(longest, &ws)) {
        delete p;
        return rc;
    }
    return finish_create(p, (n ? n : 1) * 4, ws, 4, plan);
}

extern "C" int prism_b200_host_scan_run(prism_b200_host_plan* p, uint32_t* x_host, void* stream) {
    if (int rc = check_plan(p, kScan, "host_scan_run")) return rc;
    if (p->n == 0) return PRISM_B200_OK;
    if (!x_host) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "host_scan_run: null pointer");
    cudaStream_t caller = static_cast<cudaStream_t>(stream);
    if (int rc = begin_run(p, caller)) return rc;
    uint32_t* x = static_cast<uint32_t*>(p->a);
    uint32_t* carry = static_cast<uint32_t*>(p->c);
    PRISM_RUN_TRY(cudaMemsetAsync(carry, 0, 4, p->lane[1]));
    for (size_t j = 0; j < p->blocks.size(); ++j) {
        const size_t lo = p->blocks[j].first, hi = p->blocks[j].second;
        PRISM_RUN_TRY(cudaMemcpyAsync(x + lo, x_host + lo, (hi - lo) * 4, cudaMemcpyHostToDevice, p->lane[0]));
        PRISM_RUN_TRY(cudaEventRecord(p->uploaded[j], p->lane[0]));
        PRISM_RUN_TRY(cudaStreamWaitEvent(p->lane[1], p->uploaded[j], 0));
        // seed = totals[0] with rank 1: the carry word, i.e. the scanned last element of the block before
        if (int rc = prism_b200_scan_seeded(hi - lo, x + lo, p->b, carry, 1, p->lane[1])) return abandon_run(p, caller, rc);
        PRISM_RUN_TRY(cudaMemcpyAsync(carry, x + hi - 1, 4, cudaMemcpyDeviceToDevice, p->lane[1]));
        PRISM_RUN_TRY(cudaEventRecord(p->computed[j], p->lane[1]));
        PRISM_RUN_TRY(cudaStreamWaitEvent(p->lane[2], p->computed[j], 0));
        PRISM_RUN_TRY(cudaMemcpyAsync(x_host + lo, x + lo, (hi - lo) * 4, cudaMemcpyDeviceToHost, p->lane[2]));
    }
    return end_run(p, caller);
}

extern "C" int prism_b200_host_plan_blocks(const prism_b200_host_plan* p) {
    return (p && p->magic == kMagic) ? static_cast<int>(p->blocks.size()) : -1;
}

extern "C" void prism_b200_host_plan_destroy(prism_b200_host_plan* p) {
    if (!p || p->magic != kMagic) return;
    for (auto s : p->lane)
        if (s) cudaStreamSynchronize(s);
    destroy(p);
}
