// Version / error plumbing of the atlas_b200 C ABI.
#include "common.cuh"

#include <cstring>

namespace atlas {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

void clear_error() { g_err[0] = '\0'; }

int check_cuda(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return ATLAS_OK;
    set_error("%s: %s", what, cudaGetErrorString(e));
    return ATLAS_ERR_LAUNCH;
}

int check_device() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        set_error("no CUDA device: %s", cudaGetErrorString(e));
        return ATLAS_ERR_NO_DEVICE;
    }
    static thread_local int cached_dev = -1;
    static thread_local int cached_major = 0;
    if (cached_dev != dev) {
        int major = 0;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e != cudaSuccess) {
            set_error("cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
            return ATLAS_ERR_NO_DEVICE;
        }
        cached_dev = dev;
        cached_major = major;
    }
    if (cached_major != 10) {
        set_error("device %d has compute capability %d.x; this library is built for sm_100a only",
                  dev, cached_major);
        return ATLAS_ERR_NO_DEVICE;
    }
    return ATLAS_OK;
}

}  // namespace atlas

extern "C" {

int atlas_version(void) { return 100; /* 0.1.0 */ }

const char *atlas_last_error(void) { return atlas::g_err; }

const char *atlas_status_string(int status) {
    switch (status) {
        case ATLAS_OK: return "ok";
        case ATLAS_ERR_BAD_ARGUMENT: return "bad argument";
        case ATLAS_ERR_UNSUPPORTED: return "unsupported shape or block size";
        case ATLAS_ERR_CAPACITY: return "buffer too small";
        case ATLAS_ERR_LAUNCH: return "CUDA error";
        case ATLAS_ERR_TIMEOUT: return "device-side wait timed out";
        case ATLAS_ERR_NO_DEVICE: return "no usable sm_100a device";
        default: return "unknown status";
    }
}

}  // extern "C"
