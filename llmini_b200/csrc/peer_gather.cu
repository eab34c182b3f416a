// The all-gather of packed weights as plain stores into the other GPUs' memory (one process per GPU, buffers
// shared through CUDA IPC, NVLink peer access): a rank copies its freshly encoded slice of the arena to the same
// offset of every peer's arena and then tells every peer how many such copies it has completed; a peer that needs
// the whole arena waits until every rank's count has caught up with its own.  No library collective, no launch of
// more than one small kernel per copy, so the fixed cost per bucket is a few microseconds.  Only plain loads of
// local memory and plain stores to peer memory are used: no TMA, no multicast.
//
// Control block (256 bytes behind the arena in every rank's buffer):
//   arrived[B2_MAX_PEERS]  written by the peers: arrived[p] = copies rank p has completed into this buffer
//   pushed                 copies this rank has completed into its peers (what it expects of every peer, since all
//                          ranks issue the same sequence of copies)
//   cta_done               last-CTA detection of the copy kernel
//   status                 set when the bounded wait ran out
#include <cuda_runtime.h>

#include <cstring>

#include "../../include/llmini_b200.h"

namespace {

constexpr int kPushThreads = 256;
constexpr uint32_t kCtrlArrived = 0;                        // word offsets in the control block
constexpr uint32_t kCtrlPushed = B2_MAX_PEERS;
constexpr uint32_t kCtrlCtaDone = B2_MAX_PEERS + 1;
constexpr uint32_t kCtrlStatus = B2_MAX_PEERS + 2;
constexpr size_t kCtrlBytes = 256;
static_assert((B2_MAX_PEERS + 3) * 4 <= kCtrlBytes, "control block");

struct PeerTable {
    uint64_t base[B2_MAX_PEERS];
};

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Copies [offset, offset + bytes) of this rank's buffer to the same place in every peer's buffer, then raises this
// rank's count in every peer's control block.  Every thread fences its own peer stores at system scope; the CTAs
// count themselves off (the fence / atomic / fence pattern of a last-block reduction) and the last one publishes.
__global__ void __launch_bounds__(kPushThreads)
k_peer_push(PeerTable peers, uint32_t world, uint32_t rank, size_t offset, size_t bytes, size_t ctrl_offset) {
    const uint4 *src = reinterpret_cast<const uint4 *>(peers.base[rank] + offset);
    const size_t n = bytes / 16;
    // four 16-byte pieces per thread and turn, all loads before the first store: one load's latency per 64 bytes
    // and peer would leave the links idle
    constexpr int kUnroll = 4;
    const size_t stride = (size_t)gridDim.x * kPushThreads;
    for (size_t i0 = (size_t)blockIdx.x * kPushThreads + threadIdx.x; i0 < n; i0 += kUnroll * stride) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const size_t i = i0 + u * stride;
            if (i < n) v[u] = __ldcg(src + i);   // written moments ago by the encode: mostly still in L2
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const size_t i = i0 + u * stride;
            if (i >= n) continue;
#pragma unroll
            for (uint32_t p = 0; p < B2_MAX_PEERS; ++p)
                if (p < world && p != rank) *reinterpret_cast<uint4 *>(peers.base[p] + offset + 16 * i) = v[u];
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t *ctrl = reinterpret_cast<uint32_t *>(peers.base[rank] + ctrl_offset);
        __threadfence();
        const uint32_t before = atomicAdd(ctrl + kCtrlCtaDone, 1u);
        __threadfence();
        if (before == gridDim.x - 1) {
            ctrl[kCtrlCtaDone] = 0;
            const uint32_t count = ctrl[kCtrlPushed] + 1u;
            ctrl[kCtrlPushed] = count;
            __threadfence_system();
#pragma unroll
            for (uint32_t p = 0; p < B2_MAX_PEERS; ++p)
                if (p < world && p != rank)
                    st_release_sys(reinterpret_cast<uint32_t *>(peers.base[p] + ctrl_offset) + kCtrlArrived + rank, count);
        }
    }
}

// One warp, one lane per peer: waits (bounded) until that peer's count has reached this rank's own.
__global__ void k_peer_wait(uint64_t local_base, uint32_t world, uint32_t rank, size_t ctrl_offset, uint64_t wait_ns) {
    uint32_t *ctrl = reinterpret_cast<uint32_t *>(local_base + ctrl_offset);
    const uint32_t p = threadIdx.x;
    if (p >= world || p == rank) return;
    const uint32_t want = *reinterpret_cast<volatile uint32_t *>(ctrl + kCtrlPushed);
    const uint64_t start = timer_ns();
    // counts only grow; the signed difference keeps the comparison right across a wrap
    while ((int32_t)(ld_acquire_sys(ctrl + kCtrlArrived + p) - want) < 0) {
        if (timer_ns() - start > wait_ns) {
            atomicExch(ctrl + kCtrlStatus, 1u);
            return;
        }
        __nanosleep(200);
    }
}

bool valid_group(const b2_peer_group *g) {
    return g && g->world >= 1 && g->world <= B2_MAX_PEERS && g->rank < g->world && g->base[g->rank] != 0;
}
size_t ctrl_offset_of(const b2_peer_group *g) { return (size_t)((g->arena_bytes + 255) / 256 * 256); }

}  // namespace

extern "C" {

int b2_peer_buffer_alloc(size_t arena_bytes, void **d_ptr, uint8_t handle[64]) {
    if (!d_ptr || !handle) return B2_ERROR_INVALID_VALUE;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    const size_t total = (arena_bytes + 255) / 256 * 256 + kCtrlBytes;
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, total);
    if (e != cudaSuccess) return (int)e;
    e = cudaMemset(p, 0, total);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return (int)e;
    }
    std::memcpy(handle, &h, 64);
    *d_ptr = p;
    return B2_SUCCESS;
}
int b2_peer_buffer_open(const uint8_t handle[64], void **d_ptr) {
    if (!d_ptr || !handle) return B2_ERROR_INVALID_VALUE;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, 64);
    return (int)cudaIpcOpenMemHandle(d_ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
int b2_peer_buffer_close(void *d_ptr) { return d_ptr ? (int)cudaIpcCloseMemHandle(d_ptr) : B2_SUCCESS; }
int b2_peer_buffer_free(void *d_ptr) { return d_ptr ? (int)cudaFree(d_ptr) : B2_SUCCESS; }

int b2_peer_push(const b2_peer_group *group, size_t offset, size_t bytes, uint32_t ctas, void *stream) {
    if (!valid_group(group) || offset % 16 != 0 || bytes % 16 != 0 || offset > group->arena_bytes ||
        bytes > group->arena_bytes - offset)
        return B2_ERROR_INVALID_VALUE;
    for (uint32_t p = 0; p < group->world; ++p)
        if (group->base[p] == 0 || group->base[p] % 16 != 0) return B2_ERROR_INVALID_VALUE;
    PeerTable t;
    std::memset(&t, 0, sizeof(t));
    for (uint32_t p = 0; p < group->world; ++p) t.base[p] = group->base[p];
    // enough CTAs to keep the links busy, few enough to leave the SMs to the kernels this copy runs beside
    size_t want = (bytes / 16 + 4 * kPushThreads - 1) / (4 * kPushThreads);
    if (ctas == 0) ctas = 48;
    if (want < 1) want = 1;
    const unsigned grid = (unsigned)(want < ctas ? want : ctas);
    k_peer_push<<<grid, kPushThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(t, group->world, group->rank, offset,
                                                                                  bytes, ctrl_offset_of(group));
    return (int)cudaGetLastError();
}
int b2_peer_wait(const b2_peer_group *group, uint64_t wait_ns, void *stream) {
    if (!valid_group(group)) return B2_ERROR_INVALID_VALUE;
    if (wait_ns == 0 || wait_ns > 2000000000ull) wait_ns = 2000000000ull;
    k_peer_wait<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(group->base[group->rank], group->world, group->rank,
                                                                     ctrl_offset_of(group), wait_ns);
    return (int)cudaGetLastError();
}
int b2_peer_status(const b2_peer_group *group, void *stream) {
    if (!valid_group(group)) return B2_ERROR_INVALID_VALUE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    uint32_t *word = reinterpret_cast<uint32_t *>(group->base[group->rank] + ctrl_offset_of(group)) + kCtrlStatus;
    uint32_t v = 0;
    cudaError_t e = cudaMemcpyAsync(&v, word, sizeof(v), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return (int)e;
    if (v == 0) return B2_SUCCESS;
    e = cudaMemsetAsync(word, 0, sizeof(v), s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    return e == cudaSuccess ? B2_ERROR_LAUNCH_TIMEOUT : (int)e;
}

}  // extern "C"
