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
#include "philox.h"

FR_EXPORT const char* rowwise_last_error() { return fr_error_text; }

// ------------------------------------------------------------------ embedding
// Copies one row of `width` elements; 16 bytes at a time when rows start on 16-byte boundaries.
template <typename T>
__device__ __forceinline__ void copy_row(const T* __restrict__ src, T* __restrict__ dst, int width) {
    constexpr int PER = 16 / sizeof(T);
    if (width % PER == 0 && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
        const uint4* s4 = (const uint4*)src;
        uint4* d4 = (uint4*)dst;
        for (int i = threadIdx.x; i < width / PER; i += blockDim.x) d4[i] = s4[i];
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
    }
}

// Ids are checked on the host before a step runs.  An id that a sampler chose on the device can still be outside
// the table (-1 for a row of logits without a finite entry): such a row reads nothing and becomes zeros, and the
// host, which sees the id when it reads the chosen tokens, raises.
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ tokens, const T* __restrict__ table, T* __restrict__ out,
                                 int width, int vocab) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int row = blockIdx.x;
    const int token = tokens[row];
    if (token < 0 || token >= vocab) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) fr_store(out + (size_t)row * width + i, 0.f);
        return;
    }
    copy_row(table + (size_t)token * width, out + (size_t)row * width, width);
}

FR_EXPORT int rowwise_embedding(const int* tokens, const void* table, void* out, int n_rows, int width, int vocab,
                                int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    if (dtype == FR_F32)
        embedding_kernel<float><<<n_rows, 256, 0, stream>>>(tokens, (const float*)table, (float*)out, width, vocab);
    else if (dtype == FR_BF16)
        FR_CUDA(fr_launch(embedding_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, stream, tokens,
                          (const __nv_bfloat16*)table, (__nv_bfloat16*)out, width, vocab));
    else
        FR_REFUSE("embedding: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("embedding");
    return FR_OK;
}

// ------------------------------------------------------------------ gather rows
template <typename T>
__global__ void gather_rows_kernel(const int* __restrict__ rows, const T* __restrict__ src, T* __restrict__ out,
                                   int width) {
    fr_pdl_wait();
    fr_pdl_launch();
    copy_row(src + (size_t)rows[blockIdx.x] * width, out + (size_t)blockIdx.x * width, width);
}

FR_EXPORT int rowwise_gather_rows(const int* rows, const void* src, void* out, int n_rows, int width, int dtype,
                                  cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    if (dtype == FR_F32)
        gather_rows_kernel<float><<<n_rows, 256, 0, stream>>>(rows, (const float*)src, (float*)out, width);
    else if (dtype == FR_BF16)
        FR_CUDA(fr_launch(gather_rows_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, stream, rows,
                          (const __nv_bfloat16*)src, (__nv_bfloat16*)out, width));
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
    fr_pdl_wait();
    fr_pdl_launch();
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

// bf16 rows of up to 8 * 256 * RMS_CHUNKS elements, a multiple of 8: every thread keeps its 16-byte pieces in
// registers between the sum of squares and the scaling, so the row is read once.
constexpr int RMS_CHUNKS = 4;
__global__ void __launch_bounds__(256)
rmsnorm_bf16_kernel(const __nv_bfloat16* __restrict__ x, FrVec w, __nv_bfloat16* __restrict__ y, int width, float eps) {
    __shared__ float partial[8];
    fr_pdl_wait();
    fr_pdl_launch();
    const int n_chunks = width / 8;
    const uint4* xr = (const uint4*)(x + (size_t)blockIdx.x * width);
    uint4* yr = (uint4*)(y + (size_t)blockIdx.x * width);
    uint4 v[RMS_CHUNKS];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < RMS_CHUNKS; ++i) {
        const int c = threadIdx.x + 256 * i;
        if (c < n_chunks) {
            v[i] = xr[c];
            const __nv_bfloat162* h = (const __nv_bfloat162*)&v[i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(h[j]);
                ss += f.x * f.x + f.y * f.y;
            }
        }
    }
    ss = fr_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) total += partial[i];
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
#pragma unroll
    for (int i = 0; i < RMS_CHUNKS; ++i) {
        const int c = threadIdx.x + 256 * i;
        if (c < n_chunks) {
            const __nv_bfloat16* h = (const __nv_bfloat16*)&v[i];
            uint4 o;
            __nv_bfloat16* oh = (__nv_bfloat16*)&o;
#pragma unroll
            for (int j = 0; j < 8; ++j) oh[j] = __float2bfloat16_rn(__bfloat162float(h[j]) * inv * w.at(c * 8 + j));
            yr[c] = o;
        }
    }
}

FR_EXPORT int rowwise_rmsnorm(const void* x, const void* w, int w_dtype, void* y, int n_rows, int width, float eps,
                              int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    FrVec wv{w, w_dtype};
    if (dtype == FR_F32)
        rmsnorm_kernel<float><<<n_rows, 256, 0, stream>>>((const float*)x, wv, (float*)y, width, eps);
    else if (dtype == FR_BF16 && width % 8 == 0 && width <= 8 * 256 * RMS_CHUNKS && (((uintptr_t)x | (uintptr_t)y) & 15) == 0)
        FR_CUDA(fr_launch(rmsnorm_bf16_kernel, dim3(n_rows), dim3(256), 0, stream, (const __nv_bfloat16*)x, wv,
                          (__nv_bfloat16*)y, width, eps));
    else if (dtype == FR_BF16)
        rmsnorm_kernel<__nv_bfloat16>
            <<<n_rows, 256, 0, stream>>>((const __nv_bfloat16*)x, wv, (__nv_bfloat16*)y, width, eps);
    else
        FR_REFUSE("rmsnorm: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("rmsnorm");
    return FR_OK;
}

// ------------------------------------------------------------------ SwiGLU
// gu is [rows][2*inner] with gate and up interleaved: column 2f is gate f, column 2f+1 is up f (the rows of
// the two projection matrices are stacked alternately, so that a product's tile holds both).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inner, size_t total) {
    fr_pdl_wait();
    fr_pdl_launch();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const float g = fr_load(gu + 2 * idx);
        const float u = fr_load(gu + 2 * idx + 1);
        fr_store(out + idx, g / (1.0f + expf(-g)) * u);
    }
}

FR_EXPORT int rowwise_swiglu(const void* gu, void* out, int n_rows, int inner, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    const size_t total = (size_t)n_rows * inner;
    const long long cap = (long long)(fr_sm_count() > 0 ? fr_sm_count() : 128) * 16;       // a few waves of the device
    const int blocks = (int)((long long)((total + 255) / 256) < cap ? (total + 255) / 256 : cap);
    if (dtype == FR_F32)
        swiglu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gu, (float*)out, inner, total);
    else if (dtype == FR_BF16)
        FR_CUDA(fr_launch(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gu,
                          (__nv_bfloat16*)out, inner, total));
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
    extern __shared__ float cos_sin[];           // [rot/2][2], the row's angles, shared by all heads
    // The row's sequence, position and page and the angles depend on the step's geometry alone, which is final
    // before the step's first kernel starts (common.cuh): they are taken ahead of the wait for the kernel that
    // writes qkv.
    const int row = blockIdx.x;
    const int seq = row_seq[row];
    if (seq < 0) {
        fr_pdl_wait();
        fr_pdl_launch();
        return;
    }
    const int pos = row_pos[row];
    T* base = qkv + (size_t)row * (nq + 2 * nkv) * hd;
    const int half = rot / 2;
    if (denom != nullptr) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float s, c;
            sincosf(__fdiv_rn((float)pos, denom[i]), &s, &c);
            cos_sin[2 * i] = c;
            cos_sin[2 * i + 1] = s;
        }
        __syncthreads();
    }
    T* k_dst = nullptr;
    T* v_dst = nullptr;
    if (write) {
        const int pg = block_table[(size_t)seq * table_width + pos / page];
        const size_t cache_row = ((size_t)pg * page + pos % page) * nkv * hd;
        k_dst = k_pool + cache_row;
        v_dst = v_pool + cache_row;
    }
    fr_pdl_wait();
    fr_pdl_launch();
    // The heads (q, then k, then v) are dealt out to the blocks of this row.
    const int heads = nq + 2 * nkv;
    const int per = (heads + gridDim.y - 1) / gridDim.y;
    const int h0 = blockIdx.y * per, h1 = min(h0 + per, heads);
    // q and k heads: rotate the pairs (i, i + rot/2) in place; k also goes to the cache.
    const int rot_heads = max(0, min(h1, nq + nkv) - h0);
    bool by_eights = false;
    if constexpr (sizeof(T) == 2) {
        // bf16 with 16-byte aligned heads: eight pairs per thread, as two 16-byte pieces in and two (or four) out
        by_eights = denom != nullptr && half % 8 == 0 && hd % 8 == 0 && (((uintptr_t)base) & 15) == 0 &&
                    (!write || (((uintptr_t)k_dst) & 15) == 0);
        if (by_eights) {
            const int pieces = half / 8;
            for (int idx = threadIdx.x; idx < rot_heads * pieces; idx += blockDim.x) {
                const int h = h0 + idx / pieces, i = (idx % pieces) * 8;
                T* v = base + (size_t)h * hd;
                uint4 lo = *(const uint4*)(v + i), hi = *(const uint4*)(v + i + half);
                uint32_t* lw = (uint32_t*)&lo;
                uint32_t* hw = (uint32_t*)&hi;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float ra0, rb0, ra1, rb1;
                    fr_rotate(__uint_as_float(lw[j] << 16), __uint_as_float(hw[j] << 16), cos_sin[2 * (i + 2 * j)],
                              cos_sin[2 * (i + 2 * j) + 1], ra0, rb0);
                    fr_rotate(__uint_as_float(lw[j] & 0xffff0000u), __uint_as_float(hw[j] & 0xffff0000u),
                              cos_sin[2 * (i + 2 * j + 1)], cos_sin[2 * (i + 2 * j + 1) + 1], ra1, rb1);
                    const __nv_bfloat162 a2 = __floats2bfloat162_rn(ra0, ra1), b2 = __floats2bfloat162_rn(rb0, rb1);
                    lw[j] = *(const uint32_t*)&a2;
                    hw[j] = *(const uint32_t*)&b2;
                }
                *(uint4*)(v + i) = lo;
                *(uint4*)(v + i + half) = hi;
                if (write && h >= nq) {
                    *(uint4*)(k_dst + (size_t)(h - nq) * hd + i) = lo;
                    *(uint4*)(k_dst + (size_t)(h - nq) * hd + i + half) = hi;
                }
            }
        }
    }
    if (denom != nullptr && !by_eights) {
        for (int idx = threadIdx.x; idx < rot_heads * half; idx += blockDim.x) {
            const int h = h0 + idx / half, i = idx % half;
            const float c = cos_sin[2 * i], s = cos_sin[2 * i + 1];
            T* v = base + (size_t)h * hd;
            const float a = fr_load(v + i), b = fr_load(v + i + half);
            float ra, rb;
            fr_rotate(a, b, c, s, ra, rb);
            fr_store(v + i, ra);
            fr_store(v + i + half, rb);
            if (write && h >= nq) {
                fr_store(k_dst + (size_t)(h - nq) * hd + i, ra);
                fr_store(k_dst + (size_t)(h - nq) * hd + i + half, rb);
            }
        }
    }
    if (write) {
        // what the rotation did not write: k beyond the rotated dimensions (all of k without rotation), and v
        const int k_from = denom != nullptr ? rot : 0;
        const int k_tail = hd - k_from;
        const int kh0 = max(h0, nq), kh1 = min(h1, nq + nkv);
        for (int idx = threadIdx.x; idx < max(0, kh1 - kh0) * k_tail; idx += blockDim.x) {
            const int h = kh0 + idx / k_tail, d = k_from + idx % k_tail;
            k_dst[(size_t)(h - nq) * hd + d] = base[(size_t)h * hd + d];
        }
        const int vh0 = max(h0, nq + nkv), vh1 = h1;
        constexpr int PER = 16 / sizeof(T);
        if (hd % PER == 0 && ((((uintptr_t)base) | ((uintptr_t)v_dst)) & 15) == 0) {
            const int chunks = hd / PER;
            for (int idx = threadIdx.x; idx < max(0, vh1 - vh0) * chunks; idx += blockDim.x) {
                const int h = vh0 + idx / chunks, ch = idx % chunks;
                ((uint4*)(v_dst + (size_t)(h - nq - nkv) * hd))[ch] = ((const uint4*)(base + (size_t)h * hd))[ch];
            }
        } else {
            for (int idx = threadIdx.x; idx < max(0, vh1 - vh0) * hd; idx += blockDim.x) {
                const int h = vh0 + idx / hd, d = idx % hd;
                v_dst[(size_t)(h - nq - nkv) * hd + d] = base[(size_t)h * hd + d];
            }
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
    const int heads = nq + 2 * nkv;
    const dim3 grid(n_rows, n_rows < 64 ? (heads < 4 ? heads : 4) : 1);     // few rows: spread the heads over more SMs
    const size_t smem = (size_t)(rot > 0 ? rot : 2) * sizeof(float);
    if (dtype == FR_F32)
        rope_kv_write_kernel<float><<<grid, threads, smem, stream>>>((float*)qkv, row_seq, row_pos, denom, rot, nq, nkv,
                                                                     hd, (float*)k_pool, (float*)v_pool, block_table,
                                                                     table_width, page, write);
    else if (dtype == FR_BF16)
        FR_CUDA(fr_launch(rope_kv_write_kernel<__nv_bfloat16>, grid, dim3(threads), smem, stream,
                          (__nv_bfloat16*)qkv, row_seq, row_pos, denom, rot, nq, nkv, hd, (__nv_bfloat16*)k_pool,
                          (__nv_bfloat16*)v_pool, block_table, table_width, page, write));
    else
        FR_REFUSE("rotary: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("rope_kv_write");
    return FR_OK;
}

// ------------------------------------------------------------------ advance
// After a decode step that stays on the device: the sampled token becomes the next
// input, position and length of every live row grow by one, and so does the number of
// draws made for it (the sampler's step counter), if given.
__global__ void advance_kernel(int* tokens, const int* __restrict__ sampled, int* row_pos, int* kv_len,
                               const int* __restrict__ row_seq, int* draws, int n) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (draws != nullptr) draws[i] += 1;
    if (row_seq[i] < 0) return;
    tokens[i] = sampled[i];
    row_pos[i] += 1;
    kv_len[i] += 1;
}

FR_EXPORT int rowwise_advance(int* tokens, const int* sampled, int* row_pos, int* kv_len, const int* row_seq, int* draws,
                              int n, cudaStream_t stream) {
    if (n <= 0) return FR_OK;
    FR_CUDA(fr_launch(advance_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, tokens, sampled, row_pos, kv_len,
                      row_seq, draws, n));
    FR_CHECK_LAUNCH("advance");
    return FR_OK;
}

// ------------------------------------------------------------------ multipliers, logit finish, random numbers
// x *= scale, for architectures whose token rows carry a multiplier.
template <typename T>
__global__ void scale_rows_kernel(T* x, long long n, float scale) {
    fr_pdl_wait();
    fr_pdl_launch();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        fr_store(x + i, __fmul_rn(fr_load(x + i), scale));
}

FR_EXPORT int rowwise_scale_rows(void* x, long long n, float scale, int dtype, cudaStream_t stream) {
    if (n <= 0) return FR_OK;
    const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    if (dtype == FR_F32)
        FR_CUDA(fr_launch(scale_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x, n, scale));
    else if (dtype == FR_BF16)
        FR_CUDA(fr_launch(scale_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)x, n, scale));
    else
        FR_REFUSE("scale_rows: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("scale_rows");
    return FR_OK;
}

// logits = softcap(scale * logits + bias): what a head may ask for beyond the product (a bias, a multiplier, a
// soft cap c * tanh(x / c)); each is skipped when it is not wanted (bias null, scale 1, softcap 0).
__global__ void finish_logits_kernel(float* logits, int vocab, int ld, FrVec bias, int has_bias, float scale, float softcap) {
    fr_pdl_wait();
    fr_pdl_launch();
    float* row = logits + (size_t)blockIdx.y * ld;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) {
        float v = __fmul_rn(row[i], scale);
        if (has_bias) v = __fadd_rn(v, bias.at(i));
        if (softcap > 0.f) v = __fmul_rn(softcap, tanhf(__fdiv_rn(v, softcap)));
        row[i] = v;
    }
}

FR_EXPORT int rowwise_finish_logits(float* logits, int rows, int vocab, int ld, const void* bias, int bias_dtype,
                                    float scale, float softcap, cudaStream_t stream) {
    if (rows <= 0 || vocab <= 0) return FR_OK;
    if (rows > 65535) FR_REFUSE("finish_logits: %d rows (at most 65535)", rows);
    const int bx = (vocab + 255) / 256 < 64 ? (vocab + 255) / 256 : 64;
    FR_CUDA(fr_launch(finish_logits_kernel, dim3(bx, rows), dim3(256), 0, stream, logits, vocab, ld, FrVec{bias, bias_dtype},
                      bias != nullptr ? 1 : 0, scale, softcap));
    FR_CHECK_LAUNCH("finish_logits");
    return FR_OK;
}

// out[i] = mean + std * N(0, 1)_(key, i), drawn in double, formed in fp32 and rounded once to the storage type.
template <typename T>
__global__ void random_normal_kernel(T* out, long long n, unsigned long long key, float mean, float std) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        fr_store(out + i, __fadd_rn(__fmul_rn((float)fr_normal_at(key, (uint64_t)i), std), mean));
}

FR_EXPORT int rowwise_random_normal(void* out, long long n, int dtype, unsigned long long key, float mean, float std,
                                    cudaStream_t stream) {
    if (n <= 0) return FR_OK;
    const long long cap = (long long)(fr_sm_count() > 0 ? fr_sm_count() : 128) * 32;
    const int blocks = (int)((n + 255) / 256 < cap ? (n + 255) / 256 : cap);
    if (dtype == FR_F32)
        random_normal_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, n, key, mean, std);
    else if (dtype == FR_BF16)
        random_normal_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)out, n, key, mean, std);
    else
        FR_REFUSE("random_normal: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("random_normal");
    return FR_OK;
}
