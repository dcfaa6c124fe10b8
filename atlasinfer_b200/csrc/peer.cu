// Inter-process plumbing of the column-parallel linear: device memory that the other ranks of a node can
// map (CUDA IPC over plain cudaMalloc memory), the stand-alone wait on the ranks' arrival flags, and the
// stand-alone push of a finished output shard into every rank's gathered buffer (for linears computed by a
// kernel without the fused peer-store epilogue).
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

struct PushParams {
    const unsigned char *src;
    long long rows, row_bytes, src_pitch, dst_pitch;   // bytes
    int world, rank;
    unsigned char *dst[ATLAS_MAX_PEERS];
    unsigned int *flags_dst[ATLAS_MAX_PEERS];
    unsigned int *state;
};

// Copies this rank's [rows x row_bytes] shard into every rank's gathered buffer (plain peer stores, 16 bytes per
// thread and destination, own rank first), then the CTA that finishes last publishes the arrival count.
template <typename T>
__global__ void __launch_bounds__(256) peer_push_kernel(PushParams p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the shard is the previous kernel's output
    const long long per_row = p.row_bytes / (long long)sizeof(T), total = p.rows * per_row;
    const long long stride = (long long)gridDim.x * blockDim.x;
    constexpr int U = 4;   // independent loads in flight per thread
    for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += U * stride) {
        T v[U];
        long long off[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long i = i0 + u * stride;
            off[u] = -1;
            if (i < total) {
                const long long r = i / per_row, c = i - r * per_row;
                v[u] = __ldcg(reinterpret_cast<const T *>(p.src + r * p.src_pitch) + c);
                off[u] = r * p.dst_pitch + c * (long long)sizeof(T);
            }
        }
        for (int d = 0; d < p.world; ++d) {
            int to = p.rank + d;
            if (to >= p.world) to -= p.world;
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (off[u] >= 0) *reinterpret_cast<T *>(p.dst[to] + off[u]) = v[u];
        }
    }
    // each CTA counts itself in with a release at GPU scope (the barrier orders the CTA's stores before it); the last
    // one acquires the others' releases by the same atomic and releases everything at system scope with the flag stores
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned int finished;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(finished) : "l"(p.state) : "memory");
        if (finished == gridDim.x - 1) {
            const unsigned int seq = *reinterpret_cast<volatile unsigned int *>(p.state + 1) + 1u;
            p.state[0] = 0;
            p.state[1] = seq;
            asm volatile("fence.acq_rel.sys;" ::: "memory");   // one system-scope release for all the flag stores
            for (int d = 0; d < p.world; ++d) {
                int to = p.rank + d;
                if (to >= p.world) to -= p.world;
                asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.flags_dst[to] + p.rank), "r"(seq) : "memory");
            }
        }
    }
}

template <typename K, typename... Args>
int launch_after_previous(K kern, unsigned grid, unsigned block, cudaStream_t st, const char *what, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(block, 1, 1);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // become resident while the previous kernel drains
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, args...), what);
}

}  // namespace
}  // namespace atlas

extern "C" {

int atlas_peer_push(const void *src, int64_t rows, int64_t row_bytes, int64_t src_pitch_bytes, int64_t dst_pitch_bytes,
                    const AtlasPeerGather *gather, void *stream) {
    using namespace atlas;
    clear_error();
    ATLAS_RETURN_IF(!src || !gather || rows < 0 || row_bytes <= 0 || src_pitch_bytes < row_bytes || dst_pitch_bytes < row_bytes,
                    ATLAS_ERR_BAD_ARGUMENT, "atlas_peer_push: bad argument");
    ATLAS_RETURN_IF(gather->world < 1 || gather->world > ATLAS_MAX_PEERS || gather->rank < 0 || gather->rank >= gather->world ||
                        !gather->state, ATLAS_ERR_BAD_ARGUMENT, "atlas_peer_push: bad gather descriptor");
    ATLAS_RETURN_IF((row_bytes | src_pitch_bytes | dst_pitch_bytes) & 1, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_peer_push: sizes must be even (16-bit elements)");
    PushParams p;
    p.src = (const unsigned char *)src;
    p.rows = rows;
    p.row_bytes = row_bytes;
    p.src_pitch = src_pitch_bytes;
    p.dst_pitch = dst_pitch_bytes;
    p.world = gather->world;
    p.rank = gather->rank;
    p.state = gather->state;
    bool vec = (((uintptr_t)src | (uintptr_t)row_bytes | (uintptr_t)src_pitch_bytes | (uintptr_t)dst_pitch_bytes) & 15) == 0;
    for (int d = 0; d < p.world; ++d) {
        ATLAS_RETURN_IF(!gather->y_dst[d] || !gather->flags_dst[d], ATLAS_ERR_BAD_ARGUMENT, "atlas_peer_push: null destination");
        p.dst[d] = (unsigned char *)gather->y_dst[d];
        p.flags_dst[d] = gather->flags_dst[d];
        vec = vec && ((uintptr_t)gather->y_dst[d] & 15) == 0;
    }
    int rc = check_device();
    if (rc) return rc;
    const int64_t pieces = rows * (row_bytes / (vec ? 16 : 2));
    int64_t grid = ceil_div_i64(pieces > 0 ? pieces : 1, 256 * 4);   // four pieces per thread
    if (grid > 592) grid = 592;
    if (vec) return launch_after_previous(peer_push_kernel<uint4>, (unsigned)grid, 256, (cudaStream_t)stream, "peer_push_kernel launch", p);
    return launch_after_previous(peer_push_kernel<unsigned short>, (unsigned)grid, 256, (cudaStream_t)stream, "peer_push_kernel launch", p);
}

int atlas_peer_wait(const uint32_t *flags, int world, const uint32_t *state, int64_t poll_limit, int32_t *status,
                    void *stream) {
    using namespace atlas;
    clear_error();
    ATLAS_RETURN_IF(!flags || !state || world < 1 || world > ATLAS_MAX_PEERS || poll_limit < 1, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_peer_wait: bad argument");
    int rc = check_device();
    if (rc) return rc;
    return launch_after_previous(peer_wait_kernel, 1, 32, (cudaStream_t)stream, "peer_wait_kernel launch", flags, world, state,
                                 (long long)poll_limit, (int *)status);
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
