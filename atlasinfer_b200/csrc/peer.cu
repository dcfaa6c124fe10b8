// Inter-process plumbing of the column-parallel linear: device memory that the other ranks of a node can
// map (CUDA IPC over plain cudaMalloc memory), and the stand-alone wait on the ranks' arrival flags.
//
// The reference is single-process (no torch.distributed import anywhere), so nothing here replaces a reference
// interface; the NCCL all-gather of the output shards is the baseline these calls improve on (the messages are
// 64 KB .. 1.8 MB: latency-bound, so the kernel stores its shard into the peers' buffers itself).
#include <cstring>

#include "common.cuh"

namespace atlas {
namespace {

__global__ void peer_wait_kernel(const unsigned int *flags, int world, const unsigned int *state, long long limit,
                                 int *status) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x;
    const unsigned int target = *reinterpret_cast<const volatile unsigned int *>(state + 1);
    bool ok = true;
    if (lane < world) {
        ok = false;
        for (long long i = 0; i < limit; ++i) {
            unsigned int v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + lane) : "memory");
            if ((int)(v - target) >= 0) { ok = true; break; }
            __nanosleep(64);
        }
    }
    if (!__all_sync(0xffffffffu, ok) && lane == 0 && status) atomicExch(status, 1);
}

}  // namespace
}  // namespace atlas

extern "C" {

int atlas_peer_wait(const uint32_t *flags, int world, const uint32_t *state, int64_t poll_limit, int32_t *status,
                    void *stream) {
    using namespace atlas;
    clear_error();
    ATLAS_RETURN_IF(!flags || !state || world < 1 || world > ATLAS_MAX_PEERS || poll_limit < 1, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_peer_wait: bad argument");
    int rc = check_device();
    if (rc) return rc;
    peer_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flags, world, state, (long long)poll_limit, status);
    return check_cuda(cudaGetLastError(), "peer_wait_kernel launch");
}

int atlas_peer_alloc(size_t bytes, void **ptr) {
    using namespace atlas;
    clear_error();
    ATLAS_RETURN_IF(!ptr || bytes == 0, ATLAS_ERR_BAD_ARGUMENT, "atlas_peer_alloc: bad argument");
    int rc = check_device();
    if (rc) return rc;
    void *p = nullptr;
    rc = check_cuda(cudaMalloc(&p, bytes), "cudaMalloc(peer memory)");
    if (rc) return rc;
    rc = check_cuda(cudaMemset(p, 0, bytes), "cudaMemset(peer memory)");
    if (rc) { cudaFree(p); return rc; }
    *ptr = p;
    return ATLAS_OK;
}

int atlas_peer_free(void *ptr) {
    atlas::clear_error();
    return ptr ? atlas::check_cuda(cudaFree(ptr), "cudaFree(peer memory)") : ATLAS_OK;
}

int atlas_peer_export(void *ptr, unsigned char *handle) {
    using namespace atlas;
    clear_error();
    ATLAS_RETURN_IF(!ptr || !handle, ATLAS_ERR_BAD_ARGUMENT, "atlas_peer_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == ATLAS_PEER_HANDLE_BYTES, "IPC handle size");
    cudaIpcMemHandle_t h;
    int rc = check_cuda(cudaIpcGetMemHandle(&h, ptr), "cudaIpcGetMemHandle");
    if (rc) return rc;
    memcpy(handle, &h, sizeof(h));
    return ATLAS_OK;
}

int atlas_peer_import(const unsigned char *handle, void **ptr) {
    using namespace atlas;
    clear_error();
    ATLAS_RETURN_IF(!ptr || !handle, ATLAS_ERR_BAD_ARGUMENT, "atlas_peer_import: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void *p = nullptr;
    // maps the exporting GPU's memory into this process and enables peer access from the current device
    int rc = check_cuda(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    if (rc) return rc;
    *ptr = p;
    return ATLAS_OK;
}

int atlas_peer_release(void *ptr) {
    atlas::clear_error();
    return ptr ? atlas::check_cuda(cudaIpcCloseMemHandle(ptr), "cudaIpcCloseMemHandle") : ATLAS_OK;
}

}  // extern "C"
