// Row-wise kernels of the decoder: embedding gather, RMSNorm, SwiGLU, rotary
// encoding fused with the write of keys and values into the paged cache, row
// gather, and the per-step advance of positions for decoding on the device.
//
// All arithmetic is fp32 whatever the storage type.  No fast-math: the rotation
// uses sincosf and an IEEE division, the norm a true square root and division, so
// that the fp32 path agrees with a plain implementation to rounding.
//
// What the reference does for the same steps: rmsNormKernel
// (cuda_math_kernels.cu:280-321), ropeStoreKvKernel (:363-404), silu and multiply
// (:439-480), the embedding row (transformer.cpp:958-991).  The reference's fp16
// clamps and NaN scrubbing are not reproduced.
#include "common.cuh"

FR_EXPORT const char* rowwise_last_error() { return fr_error_text; }

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ tokens, const T* __restrict__ table, T* __restrict__ out,
                                 int width) {
    const int row = blockIdx.x;
    const T* src = table + (size_t)tokens[row] * width;
    T* dst = out + (size_t)row * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
}

FR_EXPORT int rowwise_embedding(const int* tokens, const void* table, void* out, int n_rows, int width, int dtype,
                                cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    if (dtype == FR_F32)
        embedding_kernel<float><<<n_rows, 256, 0, stream>>>(tokens, (const float*)table, (float*)out, width);
    else if (dtype == FR_BF16)
        embedding_kernel<__nv_bfloat16>
            <<<n_rows, 256, 0, stream>>>(tokens, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, width);
    else
        FR_REFUSE("embedding: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("embedding");
    return FR_OK;
}

// ------------------------------------------------------------------ gather rows
template <typename T>
__global__ void gather_rows_kernel(const int* __restrict__ rows, const T* __restrict__ src, T* __restrict__ out,
                                   int width) {
    const T* s = src + (size_t)rows[blockIdx.x] * width;
    T* d = out + (size_t)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) d[i] = s[i];
}

FR_EXPORT int rowwise_gather_rows(const int* rows, const void* src, void* out, int n_rows, int width, int dtype,
                                  cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    if (dtype == FR_F32)
        gather_rows_kernel<float><<<n_rows, 256, 0, stream>>>(rows, (const float*)src, (float*)out, width);
    else if (dtype == FR_BF16)
        gather_rows_kernel<__nv_bfloat16>
            <<<n_rows, 256, 0, stream>>>(rows, (const __nv_bfloat16*)src, (__nv_bfloat16*)out, width);
    else
        FR_REFUSE("gather_rows: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("gather_rows");
    return FR_OK;
}

// ------------------------------------------------------------------ RMSNorm
// y = x * (1 / sqrt(mean(x^2) + eps)) * w, one block per row.
template <typename T>
__global__ void rmsnorm_kernel(const T* __restrict__ x, FrVec w, T* __restrict__ y, int width, float eps) {
    __shared__ float partial[32];
    const T* xr = x + (size_t)blockIdx.x * width;
    T* yr = y + (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = fr_load(xr + i);
        ss += v * v;
    }
    ss = fr_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? partial[threadIdx.x] : 0.f;
        v = fr_warp_sum(v);
        if (threadIdx.x == 0) partial[0] = v;
    }
    __syncthreads();
    const float inv = 1.0f / sqrtf(partial[0] / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) fr_store(yr + i, fr_load(xr + i) * inv * w.at(i));
}

FR_EXPORT int rowwise_rmsnorm(const void* x, const void* w, int w_dtype, void* y, int n_rows, int width, float eps,
                              int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    FrVec wv{w, w_dtype};
    if (dtype == FR_F32)
        rmsnorm_kernel<float><<<n_rows, 256, 0, stream>>>((const float*)x, wv, (float*)y, width, eps);
    else if (dtype == FR_BF16)
        rmsnorm_kernel<__nv_bfloat16>
            <<<n_rows, 256, 0, stream>>>((const __nv_bfloat16*)x, wv, (__nv_bfloat16*)y, width, eps);
    else
        FR_REFUSE("rmsnorm: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("rmsnorm");
    return FR_OK;
}

// ------------------------------------------------------------------ SwiGLU
// gu is [rows][2*inner]: gate in the first `inner` columns, up in the last.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inner, size_t total) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t row = idx / inner;
        const int col = (int)(idx - row * inner);
        const float g = fr_load(gu + row * 2 * inner + col);
        const float u = fr_load(gu + row * 2 * inner + inner + col);
        fr_store(out + idx, g / (1.0f + expf(-g)) * u);
    }
}

FR_EXPORT int rowwise_swiglu(const void* gu, void* out, int n_rows, int inner, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    const size_t total = (size_t)n_rows * inner;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (dtype == FR_F32)
        swiglu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gu, (float*)out, inner, total);
    else if (dtype == FR_BF16)
        swiglu_kernel<__nv_bfloat16>
            <<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inner, total);
    else
        FR_REFUSE("swiglu: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("swiglu");
    return FR_OK;
}

// ------------------------------------------------------------------ rotary + cache write
// qkv: [rows][(nq + 2 nkv) * hd].  For each row with row_seq >= 0:
//   q and k heads: pairs (i, i + rot/2), i < rot/2, are rotated by pos / denom[i]
//   (dimensions >= rot stay); the rotated q and k are written back in place;
//   if `write`: rotated k and v go to the row of the paged cache that holds position
//   `pos` of the row's sequence: page block_table[seq][pos / page], row pos % page.
// denom == nullptr skips the rotation (a model without rotary encoding still uses
// the cache write).  k_pool / v_pool: [pages][page][nkv][hd].
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ row_seq,
                                     const int* __restrict__ row_pos, const float* __restrict__ denom, int rot,
                                     int nq, int nkv, int hd, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                     const int* __restrict__ block_table, int table_width, int page, int write) {
    const int row = blockIdx.x;
    const int seq = row_seq[row];
    if (seq < 0) return;
    const int pos = row_pos[row];
    T* base = qkv + (size_t)row * (nq + 2 * nkv) * hd;
    size_t cache_row = 0;
    if (write) {
        const int pg = block_table[(size_t)seq * table_width + pos / page];
        cache_row = ((size_t)pg * page + pos % page) * nkv * hd;
    }
    const int half = rot / 2;
    if (denom != nullptr) {
        const int n_pairs = (nq + nkv) * half;
        for (int idx = threadIdx.x; idx < n_pairs; idx += blockDim.x) {
            const int h = idx / half, i = idx - h * half;
            float s, c;
            sincosf(__fdiv_rn((float)pos, denom[i]), &s, &c);
            T* v = base + (size_t)h * hd;
            const float a = fr_load(v + i), b = fr_load(v + i + half);
            fr_store(v + i, a * c - b * s);
            fr_store(v + i + half, a * s + b * c);
        }
        __syncthreads();
    }
    if (write) {
        const int kv = nkv * hd;
        const T* k = base + (size_t)nq * hd;
        const T* v = k + kv;
        for (int i = threadIdx.x; i < kv; i += blockDim.x) {
            k_pool[cache_row + i] = k[i];
            v_pool[cache_row + i] = v[i];
        }
    }
}

FR_EXPORT int rowwise_rope_kv_write(void* qkv, const int* row_seq, const int* row_pos, const float* denom, int rot,
                                    int nq, int nkv, int hd, void* k_pool, void* v_pool, const int* block_table,
                                    int table_width, int page, int write, int n_rows, int dtype,
                                    cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    if (rot < 0 || rot > hd || (rot & 1)) FR_REFUSE("rotary: rotary size %d must be even and at most the head size %d", rot, hd);
    if (write && (k_pool == nullptr || v_pool == nullptr || block_table == nullptr))
        FR_REFUSE("rotary: cache write asked for without a cache");
    const int threads = 256;
    if (dtype == FR_F32)
        rope_kv_write_kernel<float><<<n_rows, threads, 0, stream>>>((float*)qkv, row_seq, row_pos, denom, rot, nq, nkv,
                                                                    hd, (float*)k_pool, (float*)v_pool, block_table,
                                                                    table_width, page, write);
    else if (dtype == FR_BF16)
        rope_kv_write_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>(
            (__nv_bfloat16*)qkv, row_seq, row_pos, denom, rot, nq, nkv, hd, (__nv_bfloat16*)k_pool,
            (__nv_bfloat16*)v_pool, block_table, table_width, page, write);
    else
        FR_REFUSE("rotary: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("rope_kv_write");
    return FR_OK;
}

// ------------------------------------------------------------------ advance
// After a decode step that stays on the device: the sampled token becomes the next
// input, position and length of every live row grow by one.
__global__ void advance_kernel(int* tokens, const int* __restrict__ sampled, int* row_pos, int* kv_len,
                               const int* __restrict__ row_seq, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n || row_seq[i] < 0) return;
    tokens[i] = sampled[i];
    row_pos[i] += 1;
    kv_len[i] += 1;
}

FR_EXPORT int rowwise_advance(int* tokens, const int* sampled, int* row_pos, int* kv_len, const int* row_seq, int n,
                              cudaStream_t stream) {
    if (n <= 0) return FR_OK;
    advance_kernel<<<(n + 127) / 128, 128, 0, stream>>>(tokens, sampled, row_pos, kv_len, row_seq, n);
    FR_CHECK_LAUNCH("advance");
    return FR_OK;
}
