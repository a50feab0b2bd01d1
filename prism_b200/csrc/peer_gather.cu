// All-gather of row blocks over peer memory (NVLink / NVSwitch), one-sided: every rank PUSHES its own
// piece into the same place of every other rank's buffer with plain 16-byte stores and then raises a
// flag word there; a consumer waits (bounded) for the flags of all ranks before it reads the block.
// No collective call, no rendezvous inside a kernel, and the kernels that later read the gathered block
// (the bf16 GEMM's TMA loads) only ever touch their own GPU's memory.
//
// It serves the multi-GPU host-buffer GEMM: B is the same on every rank, each rank uploads 1/g of a
// block of B's rows over its own PCIe link and the ranks complete the block over NVLink (the reference has
// no multi-GPU path; its harness uploads all of B on its one GPU, evals/h100_bench/main.cu:105-130).
//
// Protocol (all buffers are peer-mapped, e.g. torch symmetric memory; `epoch` is the same on every rank
// and grows by one per call):
//   push   copies `bytes` from this rank's memory to dst_offset in every peer's buffer (its own copy is
//          already in place), makes the stores visible system-wide, and whichever CTA finishes last
//          stores `epoch` into flag word `flag_index` of every peer AND of this rank;
//   wait   one warp polls `count` consecutive flag words of this rank's own array until each holds a
//          value >= epoch (so a rank that is already one call ahead does no harm), for at most
//          limit_ns; a wait that runs out raises the device status and returns.
// A rank may be one call ahead of another, never two (it needs the others' flags of call e + 1 to finish
// call e + 1, and they are raised only after their call e has ended), so callers alternate between two
// destination buffers by the parity of the epoch and never overwrite data a slower rank still reads.
#include "common.cuh"

namespace prism_b200 {
namespace {

constexpr int kPushThreads = 256;

__global__ void __launch_bounds__(kPushThreads)
peer_push_kernel(const uint4* __restrict__ src, size_t vecs, unsigned char* const* peer_dst, size_t dst_offset, int world,
                 int rank, uint32_t* const* peer_flags, int flag_index, uint32_t epoch, uint32_t* done_counter) {
    // CTA b serves peer (b % (world - 1)), skipping this rank; the CTAs of one peer share the piece evenly.
    const int others = world - 1;
    const int which = static_cast<int>(blockIdx.x) % others;
    const int peer = which < rank ? which : which + 1;
    const unsigned ctas_per_peer = gridDim.x / others;
    const unsigned slice = blockIdx.x / others;
    uint4* dst = reinterpret_cast<uint4*>(peer_dst[peer] + dst_offset);
    const size_t stride = static_cast<size_t>(ctas_per_peer) * kPushThreads;
    size_t i = static_cast<size_t>(slice) * kPushThreads + threadIdx.x;
    for (; i + 3 * stride < vecs; i += 4 * stride) {   // four 16-byte loads in flight per thread
        const uint4 a = __ldcg(src + i), b = __ldcg(src + i + stride), c = __ldcg(src + i + 2 * stride),
                    d = __ldcg(src + i + 3 * stride);
        dst[i] = a;
        dst[i + stride] = b;
        dst[i + 2 * stride] = c;
        dst[i + 3 * stride] = d;
    }
    for (; i < vecs; i += stride) dst[i] = __ldcg(src + i);
    // Every thread's stores must be visible to the peers before the flag is.
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(done_counter, 1u) == gridDim.x - 1) {
            __threadfence_system();
            for (int p = 0; p < world; ++p)
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_flags[p] + flag_index), "r"(epoch) : "memory");
            *done_counter = 0;   // ready for the next push on this stream
        }
    }
}

// world == 1, or an empty piece: only the flag.
__global__ void peer_flag_kernel(uint32_t* const* peer_flags, int world, int flag_index, uint32_t epoch) {
    const int p = threadIdx.x;
    if (p < world) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_flags[p] + flag_index), "r"(epoch) : "memory");
}

__global__ void peer_wait_kernel(const uint32_t* flags, int first, int count, uint32_t epoch, unsigned long long limit_ns) {
    const int lane = threadIdx.x;
    bool ok = true;
    if (lane < count) {
        const uint32_t* f = flags + first + lane;
        const unsigned long long t0 = global_timer_ns();
        for (uint32_t spin = 1;; ++spin) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if (static_cast<int32_t>(v - epoch) >= 0) break;   // this call's flag, or a later one
            if ((spin & 63u) == 0u && global_timer_ns() - t0 > limit_ns) {
                ok = false;
                break;
            }
            __nanosleep(200);
        }
    }
    if (!__all_sync(0xffffffffu, ok) && lane == 0) raise_device_status(DEV_PEER_WAIT_TIMEOUT);
}

}  // namespace
}  // namespace prism_b200

using namespace prism_b200;

extern "C" int prism_b200_peer_push(const void* src, size_t bytes, void* const* peer_dst, size_t dst_offset, int world,
                                    int rank, uint32_t* const* peer_flags, int flag_index, uint32_t epoch,
                                    uint32_t* done_counter, void* stream) {
    if (world < 1 || world > 32 || rank < 0 || rank >= world || flag_index < 0 || epoch == 0)
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "peer_push: need 1 <= world <= 32, a rank below world, a flag index >= 0 and a non-zero epoch");
    if (!peer_flags || (bytes && (!src || !peer_dst || !done_counter)))
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "peer_push: null pointer");
    if ((reinterpret_cast<uintptr_t>(src) | dst_offset | bytes) & 15u)
        return set_error(PRISM_B200_ERR_MISALIGNED, "peer_push: src, dst_offset and bytes must be multiples of 16");
    if (int rc = bind_status_word()) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (world == 1 || bytes == 0) {
        peer_flag_kernel<<<1, 32, 0, s>>>(peer_flags, world, flag_index, epoch);
    } else {
        const size_t vecs = bytes / 16;
        // enough CTAs per peer to keep NVLink busy, not more than the piece has work for
        size_t per_peer = (vecs + 4 * kPushThreads - 1) / (4 * kPushThreads);
        const size_t cap = 296 / static_cast<size_t>(world - 1) > 0 ? 296 / static_cast<size_t>(world - 1) : 1;
        if (per_peer > cap) per_peer = cap;
        if (per_peer < 1) per_peer = 1;
        peer_push_kernel<<<static_cast<unsigned>(per_peer * (world - 1)), kPushThreads, 0, s>>>(
            static_cast<const uint4*>(src), vecs, reinterpret_cast<unsigned char* const*>(peer_dst), dst_offset, world, rank,
            peer_flags, flag_index, epoch, done_counter);
    }
    PRISM_CUDA_TRY(cudaGetLastError());
    count_launch();
    return PRISM_B200_OK;
}

extern "C" int prism_b200_peer_wait(const uint32_t* flags, int first, int count, uint32_t epoch,
                                    unsigned long long wait_limit_ns, void* stream) {
    if (!flags || first < 0 || count < 1 || count > 32 || epoch == 0)
        return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "peer_wait: need flags, first >= 0, 1 <= count <= 32 and a non-zero epoch");
    if (wait_limit_ns == 0) wait_limit_ns = kWaitLimitNs;
    if (wait_limit_ns > 600ull * kWaitLimitNs) return set_error(PRISM_B200_ERR_INVALID_ARGUMENT, "peer_wait: wait limit above 600 s");
    if (int rc = bind_status_word()) return rc;
    peer_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, first, count, epoch, wait_limit_ns);
    PRISM_CUDA_TRY(cudaGetLastError());
    count_launch();
    return PRISM_B200_OK;
}
