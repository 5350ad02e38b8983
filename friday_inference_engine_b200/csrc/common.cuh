// Shared by every kernel file: storage types, error reporting, launch checks.
//
// Each .cu file builds into a shared library of its own with a C interface.  Every
// entry point takes raw device pointers, sizes and a stream, returns 0 on success
// and a non-zero code otherwise; the text of the last error is kept per thread and
// read with <family>_last_error().  Nothing here allocates device memory: scratch
// buffers are passed in by the caller.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

enum FrDtype { FR_F32 = 0, FR_BF16 = 1 };

#define FR_OK 0
#define FR_ERR_ARG 1      // a size or option that the kernel refuses
#define FR_ERR_CUDA 2     // the CUDA runtime reported an error

static thread_local char fr_error_text[512] = "";

#define FR_REFUSE(...)                                           \
    do {                                                         \
        snprintf(fr_error_text, sizeof fr_error_text, __VA_ARGS__); \
        return FR_ERR_ARG;                                       \
    } while (0)

#define FR_CHECK_LAUNCH(what)                                                                     \
    do {                                                                                          \
        cudaError_t e_ = cudaGetLastError();                                                      \
        if (e_ != cudaSuccess) {                                                                  \
            snprintf(fr_error_text, sizeof fr_error_text, "%s: %s", what, cudaGetErrorString(e_)); \
            return FR_ERR_CUDA;                                                                   \
        }                                                                                         \
    } while (0)

#define FR_CUDA(call)                                                                              \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess) {                                                                   \
            snprintf(fr_error_text, sizeof fr_error_text, "%s: %s", #call, cudaGetErrorString(e_)); \
            return FR_ERR_CUDA;                                                                    \
        }                                                                                          \
    } while (0)

#define FR_EXPORT extern "C" __attribute__((visibility("default")))

__device__ __forceinline__ float fr_load(const float* p) { return *p; }
__device__ __forceinline__ float fr_load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void fr_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void fr_store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// A vector of [n] that may be stored as fp32 or bf16 whatever the activations are
// (norm weights, biases): read through this.
struct FrVec {
    const void* p;
    int dtype;
    __device__ __forceinline__ float at(int i) const {
        return dtype == FR_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
    }
};

__device__ __forceinline__ float fr_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float fr_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
