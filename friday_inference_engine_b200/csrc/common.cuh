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
#include <stdlib.h>

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

// SMs of the current device (asked once per device); 0 if the query fails.
static inline int fr_sm_count() {
    static int counts[64] = {0};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
    if (counts[device] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) == cudaSuccess) counts[device] = n;
    }
    return counts[device];
}

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

// The rotation of one pair of a rotary encoding, the same instructions wherever it is applied.
__device__ __forceinline__ void fr_rotate(float a, float b, float c, float s, float& ra, float& rb) {
    ra = __fmaf_rn(-b, s, __fmul_rn(a, c));
    rb = __fmaf_rn(a, s, __fmul_rn(b, c));
}

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

// ------------------------------------------------------------------ programmatic dependent launch
// Every kernel of this library is launched so that it may start while its predecessor in
// the stream is still draining (the launch itself, block scheduling and any prologue that
// reads nothing the predecessor writes overlap with the predecessor's tail).  The contract
// inside a kernel: fr_pdl_wait() before the first access to memory that an earlier kernel
// may write or read; fr_pdl_launch() once the next kernel may be scheduled.  A kernel that
// follows one of these in a stream but was launched the ordinary way is fully serialised,
// as always.  FRIDAY_PDL=0 in the environment switches the launch attribute off.
//
// What may be read ahead of the wait: memory that only copies from the host write (page tables), and the
// geometry of the step (rows, positions, ended sequences), which is final before the step's first kernel
// starts.  The latter holds because the row-wise kernels that open every step (embedding, the first norm)
// wait before they let their dependents launch: whatever runs after them was launched after the step before
// had finished.  Kernels that let dependents launch before their own wait (the products) never open a step.
__device__ __forceinline__ void fr_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void fr_pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline bool fr_pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("FRIDAY_PDL");
        v = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

// cluster_x > 1 launches thread-block clusters of that many CTAs along x (grid.x must be a multiple of it).
template <typename... KArgs, typename... Args>
static inline cudaError_t fr_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                            cudaStream_t stream, unsigned cluster_x, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (fr_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename... KArgs, typename... Args>
static inline cudaError_t fr_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
    return fr_launch_cluster(kernel, grid, block, smem, stream, 1u, args...);
}

// Thread-block clusters: rank of this CTA, a barrier over the cluster, and a load from another CTA's shared memory.
__device__ __forceinline__ uint32_t fr_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void fr_cluster_sync() {
    asm volatile("barrier.cluster.arrive.aligned;\nbarrier.cluster.wait.aligned;" ::: "memory");
}
__device__ __forceinline__ float fr_cluster_load(const float* local, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ float4 fr_cluster_load4(const float* local, uint32_t rank) {      // 16-byte aligned
    uint32_t remote;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}
