// Peer memory for one node with one process per GPU: buffers that other ranks map through CUDA IPC
// and write into directly over NVLink (plain st.global, no multicast), and the bounded flag barrier
// that orders those writes before the kernels that read them.
//
// The reference has no multi-GPU code; these calls serve the tensor-parallel OPT layer, whose pack and
// linear kernels store their results straight into the buffers of the ranks that consume them.
#include <cuda_runtime.h>
#include <string.h>

#include "common.cuh"

namespace bsi {

// Status word of the barrier kernels (this file is compiled on its own, without relocatable device
// code, so it keeps its own word; bsi_b200_device_status reads both).
__device__ int g_peer_status = 0;

int take_peer_status(int* v) {
    int s = 0;
    BSI_CUDA_TRY(cudaMemcpyFromSymbol(&s, g_peer_status, sizeof(int)));
    if (s != 0) {
        const int zero = 0;
        BSI_CUDA_TRY(cudaMemcpyToSymbol(g_peer_status, &zero, sizeof(int)));
    }
    *v = s;
    return BSI_OK;
}

namespace {

struct FlagTable {
    uint32_t* flags[BSI_B200_MAX_PEERS];   // flags[r]: rank r's flag array (own memory for r == rank)
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// One thread per rank. The epoch is kept on the device (slot n of the rank's own flag array is the
// number of barriers passed), so a captured launch can be replayed: every rank runs the same sequence
// of barriers and the counters stay equal. Thread p tells rank p "rank `rank` reached `epoch`", then
// waits until rank p has said the same here. The fence before the signal orders every earlier write
// of this GPU (the producer kernels finished before this kernel started) ahead of the flag; the
// acquire load on the other side orders the flag ahead of the consumer kernels. The wait gives up after
// timeout_ns, records status 64 + p and returns: a missing rank must not hang the GPU.
__global__ void peer_barrier_kernel(FlagTable t, int rank, int n, unsigned long long timeout_ns) {
    __shared__ uint32_t epoch_s;
    // Deliberately a plain launch, without programmatic dependent launch: a dependent kernel that becomes
    // resident early holds its SMs while this kernel waits for other GPUs, and with two streams per rank the
    // ranks can then starve each other's producers (seen as barrier timeouts, status 64 + rank).
    uint32_t* own = t.flags[rank];
    if (threadIdx.x == 0) {
        epoch_s = own[n] + 1u;
        own[n] = epoch_s;
    }
    __syncthreads();
    const uint32_t epoch = epoch_s;
    const int p = threadIdx.x;
    if (p >= n) return;
    __threadfence_system();
    uint32_t* remote = t.flags[p] + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const uint32_t* mine = own + p;
    const unsigned long long start = global_timer_ns();
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if (static_cast<int32_t>(v - epoch) >= 0) break;
        if (global_timer_ns() - start > timeout_ns) {
            atomicCAS(&g_peer_status, 0, 64 + p);
            break;
        }
        __nanosleep(200);
    }
}

}  // namespace
}  // namespace bsi

extern "C" int bsi_b200_peer_alloc(int64_t bytes, void** dev_ptr, void* handle64) {
    using namespace bsi;
    static_assert(sizeof(cudaIpcMemHandle_t) == BSI_B200_PEER_HANDLE_BYTES, "IPC handle size");
    if (bytes <= 0 || dev_ptr == nullptr || handle64 == nullptr) return fail(BSI_ERR_INVALID, "peer_alloc: bad argument");
    void* p = nullptr;
    BSI_CUDA_TRY(cudaMalloc(&p, static_cast<size_t>(bytes)));
    cudaError_t e = cudaMemset(p, 0, static_cast<size_t>(bytes));
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle64), p);
    if (e != cudaSuccess) {
        cudaFree(p);
        set_error("peer_alloc: %s", cudaGetErrorString(e));
        return BSI_ERR_CUDA;
    }
    *dev_ptr = p;
    return BSI_OK;
}

extern "C" int bsi_b200_peer_free(void* dev_ptr) {
    using namespace bsi;
    if (dev_ptr == nullptr) return BSI_OK;
    BSI_CUDA_TRY(cudaFree(dev_ptr));
    return BSI_OK;
}

extern "C" int bsi_b200_peer_open(const void* handle64, void** peer_ptr) {
    using namespace bsi;
    if (handle64 == nullptr || peer_ptr == nullptr) return fail(BSI_ERR_INVALID, "peer_open: bad argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    void* p = nullptr;
    BSI_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *peer_ptr = p;
    return BSI_OK;
}

extern "C" int bsi_b200_peer_close(void* peer_ptr) {
    using namespace bsi;
    if (peer_ptr == nullptr) return BSI_OK;
    BSI_CUDA_TRY(cudaIpcCloseMemHandle(peer_ptr));
    return BSI_OK;
}

extern "C" int bsi_b200_peer_barrier(uint32_t* const* flags, int rank, int n, int64_t timeout_ms,
                                     bsi_stream_t stream_) {
    using namespace bsi;
    if (flags == nullptr || n < 1 || n > BSI_B200_MAX_PEERS || rank < 0 || rank >= n)
        return fail(BSI_ERR_INVALID, "peer_barrier: bad rank / n");
    if (timeout_ms <= 0) return fail(BSI_ERR_INVALID, "peer_barrier: timeout must be positive");
    FlagTable t = {};
    for (int i = 0; i < n; ++i) {
        if (flags[i] == nullptr) return fail(BSI_ERR_INVALID, "peer_barrier: null flag pointer");
        t.flags[i] = flags[i];
    }
    if (int rc = require_sm100()) return rc;
    peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(
        t, rank, n, static_cast<unsigned long long>(timeout_ms) * 1000000ull);
    return check_launch("peer_barrier launch");
}
