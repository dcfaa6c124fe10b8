// Shared host/device helpers for the atlas_b200 C-ABI library.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "atlas_b200.h"

namespace atlas {

// Thread-local text behind atlas_last_error().
void set_error(const char *fmt, ...);
void clear_error();

// Returns ATLAS_OK, or records `what` + the CUDA error text and returns ATLAS_ERR_LAUNCH.
int check_cuda(cudaError_t e, const char *what);

// ATLAS_OK if the current device is compute capability 10.x, else ATLAS_ERR_NO_DEVICE.
int check_device();

__host__ __device__ inline int64_t ceil_div_i64(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace atlas

#define ATLAS_RETURN_IF(cond, code, ...)      \
    do {                                      \
        if (cond) {                           \
            atlas::set_error(__VA_ARGS__);    \
            return (code);                    \
        }                                     \
    } while (0)
