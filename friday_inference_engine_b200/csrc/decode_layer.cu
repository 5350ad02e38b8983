// One-token steps of a stack of pre-norm decoder layers (RMSNorm -> grouped-query attention with rotary
// encoding -> residual; RMSNorm -> SwiGLU feed-forward -> residual) as ONE persistent kernel for up to 16 rows.
//
// Why: at a handful of rows every matrix product of a layer streams its weights in a few microseconds, and a
// layer run as eight or nine separate kernels spends as long again on what lies between them (set-up, the
// first dependent load, drain and flush).  Here one CTA per SM stays resident for all layers; the phases of a
// layer are separated by grid-wide barriers (an atomic counter per barrier, bounded spins) instead of kernel
// boundaries, and the warp that feeds the tensor cores never stops at a barrier for weights: it keeps the
// shared-memory ring full of the next product's weight tiles while the other warps are still normalising,
// rotating or attending.  Only loads of activations wait for the phase that produces them.
//
// Roles in a CTA (192 threads): warp 0, one lane: TMA producer for all products of all layers; warp 1, one
// lane: tcgen05.mma issuer; warps 2-5: "workers" - RMSNorm rows, the epilogues of the products (TMEM ->
// registers -> bias / residual / SwiGLU -> global, split-k merged by the last CTA to arrive), rotary encoding
// with the cache write, attention over the paged cache (mma.sync, 64-key blocks by cp.async, splits merged by
// the last CTA to arrive), and the grid barriers.
//
// Phases of a layer, each followed by a grid barrier:
//   norm1 (x -> xn) | qkv = Wqkv xn + b | rotate q, k; write k, v to the cache | attention -> attn |
//   x += Wo attn | norm2 (x -> xn) | act = silu(Wg xn) * (Wu xn) | x += Wd act
// The products use the orientation of the skinny GEMM: weights on the M side (tiles of 128 rows), the rows of
// the step as a 16-wide N tile, k cut into `splits` ranges when there are fewer tiles than SMs.
//
// The arithmetic of every phase is that of the stand-alone kernels (rowwise.cu, gemm_tc.cu, attention_mma.cu);
// the reference runs the same chain as a CUDA graph of separate kernels (transformer.cpp:997-1074, 1465-1483).
#include <cuda.h>
#include <math.h>

#include "common.cuh"
#include "tc_common.cuh"

FR_EXPORT const char* decode_layer_last_error() { return fr_error_text; }

namespace {

using namespace tc;
typedef __nv_bfloat16 bf16;

constexpr int BN = 16;                              // rows of a step, padded: N of the instruction
constexpr int STAGES = 8;
constexpr int Q_BYTES = BN * TILE_K * 2;
constexpr int STAGE_BYTES = P_BYTES + Q_BYTES;      // 18 KB
constexpr int THREADS = 192;
constexpr int WORKERS = 128;
constexpr int KEYS = 64;                            // keys per attention block = tokens per cache page
constexpr int BARRIERS_PER_LAYER = 8;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

struct GemmPhase {
    CUtensorMap map_w;      // weights [n][k], box 64 x 128
    CUtensorMap map_x;      // activations [rows][k], box 64 x 16
    void* out;              // [rows][ldo] bf16
    const void* bias;
    const void* residual;
    int bias_dtype, n, ldo, act, tiles, splits, kb_total, kb_per;
};

struct LayerArgs {
    GemmPhase qkv, o, gu, down;
    const void* norm1_w;
    const void* norm2_w;
    bf16* k_pool;           // this layer's cache entry [pages][64][nkv][hd]
    bf16* v_pool;
    const int* block_table; // [rows][table_width] of the entry's group
    const float* rope_denom;
    int norm1_dtype, norm2_dtype, table_width, window, rot;
    float eps1, eps2;
};

struct StepArgs {
    const LayerArgs* layers;
    bf16* x;                // [rows][width] residual stream, in and out
    bf16* xn;               // [rows][width]
    bf16* qkv;              // [rows][(nq + 2 nkv) hd]
    bf16* attn;             // [rows][nq hd]
    const int* row_seq;     // [rows]; negative: the row's sequence has ended
    const int* row_pos;     // [rows]
    float* gemm_scratch;    // split-k partial tiles
    int* gemm_counters;
    float* attn_scratch;    // [rows * nq][attn_splits][hd + 2]
    int* attn_counters;     // [rows * nkv * row tiles]
    int* grid_bars;         // [3]: arrivals, barriers completed, CTAs that have left; all zero between launches
    int* status;
    unsigned long long* trace;  // may be null; else [n_layers * 8 + 1] times (ns) at which CTA 0 left each grid barrier
    int n_layers, rows, width, nq, nkv, attn_splits;
    float scale_log2;
};

// What finish16 reads.
struct Epi {
    void* out;
    const void* bias;
    const void* residual;
    int p_rows, q_rows, ldo, out_dtype, bias_dtype, swapped, act;
};

__device__ __forceinline__ void worker_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// ------------------------------------------------------------------ grid barrier (workers only)
// grid_bars[0] counts arrivals, grid_bars[1] is the number of barriers that have been completed.  The last CTA
// to arrive clears the count and publishes the next number; the others watch only that second word, so the
// arrivals (atomics on word 0) and the watching (loads of word 1) do not fight over one address.  Spins are
// bounded and give up as soon as any CTA has recorded a failure.  Both words are zero between launches: the
// last CTA to leave the kernel clears the second.
__device__ bool grid_barrier(const StepArgs& a, int g, int wt, volatile int* passed) {
    __shared__ int ok_flag;
    worker_sync();
    if (wt == 0) {
        int ok = 1;
        __threadfence();
        asm volatile("fence.proxy.async;" ::: "memory");      // writes of this phase, for later TMA loads elsewhere
        const int n = (int)gridDim.x;
        if (atomicAdd(a.grid_bars, 1) == n - 1) {
            a.grid_bars[0] = 0;
            __threadfence();
            atomicExch(a.grid_bars + 1, g + 1);
        } else {
            const unsigned long long t0 = global_ns();
            for (uint32_t it = 0;; ++it) {
                if (ld_acquire(a.grid_bars + 1) > g) break;
                if ((it & 255u) == 255u) {
                    if (ld_acquire(a.status) != 0) { ok = 0; break; }
                    if (global_ns() - t0 > WAIT_LIMIT_NS) { atomicCAS(a.status, 0, 16 + (g & 15)); ok = 0; break; }
                }
            }
        }
        __threadfence();
        asm volatile("fence.proxy.async;" ::: "memory");
        ok_flag = ok;
        *passed = g + 1;                                      // the producer warp polls this
        if (a.trace != nullptr && blockIdx.x == 0) a.trace[g + 1] = global_ns();
    }
    worker_sync();
    return ok_flag != 0;
}

// ------------------------------------------------------------------ RMSNorm of one row by the 128 workers
// Rows of up to 8192 elements, a multiple of 8, are read once in 16-byte pieces and kept in registers.
__device__ void norm_row(const bf16* __restrict__ x, FrVec w, bf16* __restrict__ y, int width, float eps, int wt,
                         float* red) {
    constexpr int MAXC = 8;
    const bool vec = width % 8 == 0 && width <= 8 * WORKERS * MAXC && ((((uintptr_t)x) | ((uintptr_t)y)) & 15) == 0;
    uint4 v[MAXC];
    float ss = 0.f;
    if (vec) {
        const int n_chunks = width / 8;
#pragma unroll
        for (int i = 0; i < MAXC; ++i) {
            const int c = wt + WORKERS * i;
            if (c < n_chunks) v[i] = __ldcg((const uint4*)x + c);     // written by other SMs a moment ago: from L2
        }
#pragma unroll
        for (int i = 0; i < MAXC; ++i) {
            const int c = wt + WORKERS * i;
            if (c < n_chunks) {
                const __nv_bfloat162* h = (const __nv_bfloat162*)&v[i];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(h[j]);
                    ss += f.x * f.x + f.y * f.y;
                }
            }
        }
    } else {
        for (int i = wt; i < width; i += WORKERS) {
            const float f = __bfloat162float(x[i]);
            ss += f * f;
        }
    }
    ss = fr_warp_sum(ss);
    if ((wt & 31) == 0) red[wt >> 5] = ss;
    worker_sync();
    const float inv = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)width + eps);
    if (vec) {
        const int n_chunks = width / 8;
#pragma unroll
        for (int i = 0; i < MAXC; ++i) {
            const int c = wt + WORKERS * i;
            if (c < n_chunks) {
                const bf16* h = (const bf16*)&v[i];
                uint4 o;
                bf16* oh = (bf16*)&o;
#pragma unroll
                for (int j = 0; j < 8; ++j) oh[j] = __float2bfloat16_rn(__bfloat162float(h[j]) * inv * w.at(c * 8 + j));
                ((uint4*)y)[c] = o;
            }
        }
    } else {
        for (int i = wt; i < width; i += WORKERS) y[i] = __float2bfloat16_rn(__bfloat162float(x[i]) * inv * w.at(i));
    }
    worker_sync();
}

// ------------------------------------------------------------------ rotary encoding and cache write, one head
__device__ void rope_head(const StepArgs& a, const LayerArgs& L, int row, int h, int hd, int wt) {
    const int seq = a.row_seq[row];
    if (seq < 0) return;
    const int pos = a.row_pos[row];
    bf16* base = a.qkv + (size_t)row * (a.nq + 2 * a.nkv) * hd + (size_t)h * hd;
    const int pg = L.block_table[(size_t)row * L.table_width + pos / KEYS];
    const size_t cache_row = ((size_t)pg * KEYS + pos % KEYS) * a.nkv * hd;
    const int half = L.rot / 2;
    if (h < a.nq + a.nkv) {
        bf16* kd = h >= a.nq ? L.k_pool + cache_row + (size_t)(h - a.nq) * hd : nullptr;
        for (int i = wt; i < half; i += WORKERS) {
            float s, c;
            sincosf(__fdiv_rn((float)pos, L.rope_denom[i]), &s, &c);
            const float x0 = __bfloat162float(base[i]), x1 = __bfloat162float(base[i + half]);
            const bf16 r0 = __float2bfloat16_rn(x0 * c - x1 * s), r1 = __float2bfloat16_rn(x0 * s + x1 * c);
            base[i] = r0;
            base[i + half] = r1;
            if (kd) { kd[i] = r0; kd[i + half] = r1; }
        }
        if (kd) for (int d = L.rot + wt; d < hd; d += WORKERS) kd[d] = base[d];
    } else {
        bf16* vd = L.v_pool + cache_row + (size_t)(h - a.nq - a.nkv) * hd;
        for (int d = wt; d < hd; d += WORKERS) vd[d] = base[d];
    }
}

// ------------------------------------------------------------------ attention of one (row, kv head, row tile, split)
// The four worker warps take 16 keys each of every 64-key block; see attention_mma.cu (keys mode) for the scheme.
template <int HD>
__device__ void attention_item(const StepArgs& a, const LayerArgs& L, int row, int kvh, int tile, int split,
                               uint8_t* smem_attn, int wt) {
    constexpr int ROW_BYTES = HD * 2 + 16;
    constexpr int CHUNKS = HD / 8;
    constexpr int DT = HD / 8;
    constexpr int KV_BYTES = KEYS * ROW_BYTES;
    uint8_t* s_q = smem_attn;
    uint8_t* s_k = s_q + 16 * ROW_BYTES;
    uint8_t* s_v = s_k + 2 * KV_BYTES;
    const int warp = wt >> 5, lane = wt & 31;
    const int G = a.nq / a.nkv;
    const int r0 = tile * 16;
    const bool live = a.row_seq[row] >= 0;
    const int pos = a.row_pos[row];
    const int lo_min = L.window > 0 ? max(0, pos - L.window + 1) : 0;
    int kb_begin = lo_min / KEYS, kb_end = pos / KEYS;
    const int S = a.attn_splits;
    if (S > 1) {
        const int n = kb_end - kb_begin + 1, per = (n + S - 1) / S;
        kb_begin += split * per;
        kb_end = min(kb_begin + per - 1, kb_end);
    }
    if (!live) kb_end = kb_begin - 1;
    const int* table = L.block_table + (size_t)row * L.table_width;
    const size_t kv_row = (size_t)a.nkv * HD;
    const int q_stride = (a.nq + 2 * a.nkv) * HD;

    worker_sync();                                          // the buffers may still be read by the item before
    for (int c = wt; c < 16 * CHUNKS; c += WORKERS) {
        const int r = c / CHUNKS, ch = c - r * CHUNKS;
        const bool ok = r0 + r < G;
        const bf16* src = a.qkv + (size_t)row * q_stride + (size_t)(kvh * G + (ok ? r0 + r : 0)) * HD + ch * 8;
        cp_async16((uint32_t)__cvta_generic_to_shared(s_q + r * ROW_BYTES + ch * 16), src, ok ? 16 : 0);
    }
    auto load_kv = [&](int kb, int buf) {
        const int page = table[kb];
        const bf16* kbase = L.k_pool + ((size_t)page * KEYS) * kv_row + (size_t)kvh * HD;
        const bf16* vbase = L.v_pool + ((size_t)page * KEYS) * kv_row + (size_t)kvh * HD;
        const int valid = pos - kb * KEYS + 1;
        for (int c = wt; c < KEYS * CHUNKS; c += WORKERS) {
            const int r = c / CHUNKS, ch = c - r * CHUNKS;
            const bool ok = r < valid;
            const size_t off = (size_t)r * kv_row + ch * 8;
            cp_async16((uint32_t)__cvta_generic_to_shared(s_k + buf * KV_BYTES + r * ROW_BYTES + ch * 16),
                       ok ? (const void*)(kbase + off) : (const void*)L.k_pool, ok ? 16 : 0);
            cp_async16((uint32_t)__cvta_generic_to_shared(s_v + buf * KV_BYTES + r * ROW_BYTES + ch * 16),
                       ok ? (const void*)(vbase + off) : (const void*)L.v_pool, ok ? 16 : 0);
        }
    };
    if (kb_begin <= kb_end) load_kv(kb_begin, 0);
    cp_commit();

    const int key_base = warp * 16;
    const int rr_lo = r0 + (lane >> 2), rr_hi = rr_lo + 8;
    const bool row_ok[2] = {rr_lo < G, rr_hi < G};
    const int lo_r = L.window > 0 ? max(0, pos - L.window + 1) : 0;
    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; ++d)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[d][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(s_q);
    int buf = 0;
    for (int kb = kb_begin; kb <= kb_end; ++kb, buf ^= 1) {
        if (kb < kb_end) {
            load_kv(kb + 1, buf ^ 1);
            cp_commit();
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        worker_sync();
        const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(s_k + buf * KV_BYTES);
        const uint32_t v_addr = (uint32_t)__cvta_generic_to_shared(s_v + buf * KV_BYTES);
        float s[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            uint32_t qa[4], b[4];
            ldsm4(qa, q_addr + ((lane & 7) + 8 * ((lane >> 3) & 1)) * ROW_BYTES + (ks * 16 + 8 * (lane >> 4)) * 2);
            ldsm4(b, k_addr + (key_base + (lane & 7) + 8 * (lane >> 4)) * ROW_BYTES + (ks * 16 + 8 * ((lane >> 3) & 1)) * 2);
            mma16816(s[0], qa, b[0], b[1]);
            mma16816(s[1], qa, b[2], b[3]);
        }
        const int j0 = kb * KEYS + key_base;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = j0 + n * 8 + 2 * (lane & 3) + (e & 1);
                float v = s[n][e] * a.scale_log2;
                if (!row_ok[e >> 1] || j > pos || j < lo_r) v = -INFINITY;
                s[n][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        float alpha[2], m_use[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            const float m_new = fmaxf(m_run[i], mx[i]);
            m_use[i] = m_new == -INFINITY ? 0.f : m_new;
            alpha[i] = exp2f(m_run[i] - m_use[i]);
            m_run[i] = m_new;
        }
        float sum[2] = {0.f, 0.f};
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pe = exp2f(s[n][e] - m_use[e >> 1]);
                s[n][e] = pe;
                sum[e >> 1] += pe;
            }
#pragma unroll
        for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * alpha[i] + sum[i];
#pragma unroll
        for (int d = 0; d < DT; ++d) {
            o[d][0] *= alpha[0]; o[d][1] *= alpha[0];
            o[d][2] *= alpha[1]; o[d][3] *= alpha[1];
        }
        uint32_t pa[4];
        pa[0] = pack_bf16(s[0][0], s[0][1]);
        pa[1] = pack_bf16(s[0][2], s[0][3]);
        pa[2] = pack_bf16(s[1][0], s[1][1]);
        pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int dp = 0; dp < DT / 2; ++dp) {
            uint32_t b[4];
            ldsm4_t(b, v_addr + (key_base + (lane & 7) + 8 * ((lane >> 3) & 1)) * ROW_BYTES + (dp * 16 + 8 * (lane >> 4)) * 2);
            mma16816(o[2 * dp], pa, b[0], b[1]);
            mma16816(o[2 * dp + 1], pa, b[2], b[3]);
        }
        worker_sync();
    }
    cp_wait<0>();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
    // merge the four warps through shared memory (the K/V buffers are free now)
    float* c_o = reinterpret_cast<float*>(s_k);             // [4][16][HD]
    float* c_m = c_o + 4 * 16 * HD;
    float* c_l = c_m + 64;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = (lane >> 2) + 8 * i;
#pragma unroll
        for (int d = 0; d < DT; ++d) {
            c_o[(warp * 16 + r) * HD + d * 8 + 2 * (lane & 3)] = o[d][2 * i];
            c_o[(warp * 16 + r) * HD + d * 8 + 2 * (lane & 3) + 1] = o[d][2 * i + 1];
        }
        if ((lane & 3) == 0) {
            c_m[warp * 16 + r] = m_run[i];
            c_l[warp * 16 + r] = l_run[i];
        }
    }
    worker_sync();
    const int r = wt >> 3;
    const bool valid = r0 + r < G;
    const int h = kvh * G + (valid ? r0 + r : 0);
    const size_t item = (size_t)row * a.nq + h;
    if (valid) {
        float big = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) big = fmaxf(big, c_m[w * 16 + r]);
        float f[4], l = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            f[w] = c_m[w * 16 + r] == -INFINITY ? 0.f : exp2f(c_m[w * 16 + r] - big);
            l += c_l[w * 16 + r] * f[w];
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
        for (int d = (wt & 7); d < HD; d += 8) {
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) acc += c_o[(w * 16 + r) * HD + d] * f[w];
            if (S == 1) a.attn[item * HD + d] = __float2bfloat16_rn(acc * inv);
            else a.attn_scratch[(item * S + split) * (HD + 2) + d] = acc;
        }
        if (S > 1 && (wt & 7) == 0) {
            float* dst = a.attn_scratch + (item * S + split) * (HD + 2);
            dst[HD] = big * LN2;
            dst[HD + 1] = l;
        }
    }
    if (S > 1) {
        __shared__ int s_last;
        __threadfence();
        worker_sync();
        if (wt == 0) {
            int* c = a.attn_counters + ((size_t)row * a.nkv + kvh) * ((G + 15) / 16) + tile;
            s_last = atomicAdd(c, 1) == S - 1;
            if (s_last) *c = 0;
        }
        worker_sync();
        if (s_last) {
            __threadfence();
            const float* base = a.attn_scratch + item * S * (HD + 2);
            float* weight = c_o;
            float big = -INFINITY;
            if (valid)
                for (int sp = wt & 7; sp < S; sp += 8) big = fmaxf(big, __ldcg(base + (size_t)sp * (HD + 2) + HD));
#pragma unroll
            for (int o2 = 1; o2 < 8; o2 <<= 1) big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, o2));
            float l = 0.f;
            if (valid)
                for (int sp = wt & 7; sp < S; sp += 8) {
                    const float ls = __ldcg(base + (size_t)sp * (HD + 2) + HD + 1);
                    const float f = ls > 0.f ? expf(__ldcg(base + (size_t)sp * (HD + 2) + HD) - big) : 0.f;
                    weight[r * S + sp] = f;
                    l += ls * f;
                }
#pragma unroll
            for (int o2 = 1; o2 < 8; o2 <<= 1) l += __shfl_xor_sync(0xffffffffu, l, o2);
            __syncwarp();
            if (valid) {
                constexpr int PER = HD / 8;
                const int d0 = (wt & 7) * PER;
                float acc[PER];
#pragma unroll
                for (int i = 0; i < PER; ++i) acc[i] = 0.f;
#pragma unroll 4
                for (int sp = 0; sp < S; ++sp) {
                    const float* ps = base + (size_t)sp * (HD + 2) + d0;
                    const float f = weight[r * S + sp];
#pragma unroll
                    for (int i = 0; i < PER; ++i) acc[i] += __ldcg(ps + i) * f;
                }
                const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
                for (int i = 0; i < PER; ++i) a.attn[item * HD + d0 + i] = __float2bfloat16_rn(acc[i] * inv);
            }
        }
    }
}

// ------------------------------------------------------------------ the kernel
template <int HD>
__global__ void __launch_bounds__(THREADS, 1) decode_layers_kernel(const StepArgs a) {
    constexpr int ATTN_BYTES = 16 * (HD * 2 + 16) + 4 * KEYS * (HD * 2 + 16);
    constexpr int TMEM_COLS = 32;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_attn = smem + STAGES * STAGE_BYTES;
    uint64_t* bars = (uint64_t*)(smem_attn + ((ATTN_BYTES + 15) & ~15));
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    int* flags = (int*)(tmem_slot + 1);             // [0] split-k: came last; [1] grid barriers passed; [2..5] sums
    volatile int* passed = flags + 1;
    float* red = (float*)(flags + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t accf0 = smem_u32(bars + 2 * STAGES), acce0 = smem_u32(bars + 2 * STAGES + 2);
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(accf0 + 8 * i, 1);
            mbar_init(acce0 + 8 * i, 4);
        }
        flags[0] = 0;
        flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) fr_pdl_launch();
    const int grid = (int)gridDim.x;

    if (warp == 0) {
        if (lane == 0) {
            // All products of all layers, in order.  A stage gets its weight slice as soon as it is free; its
            // activation slice follows once the phase that writes the activations lies behind a grid barrier
            // that this CTA's workers have passed.  Until then the stages filled with weights only are "owed".
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            bool first_pass = true;                    // the ring has not wrapped yet: its stages are free
            int owed_kb[STAGES];
            fr_pdl_wait();
            for (int l = 0; l < a.n_layers && ok; ++l) {
                const LayerArgs& L = a.layers[l];
                for (int ph = 0; ph < 4 && ok; ++ph) {
                    const GemmPhase& g = ph == 0 ? L.qkv : ph == 1 ? L.o : ph == 2 ? L.gu : L.down;
                    const int need = l * BARRIERS_PER_LAYER + (ph == 0 ? 1 : ph == 1 ? 4 : ph == 2 ? 6 : 7);
                    bool go = false;
                    int owed = 0, owed_first = stage;  // stages owed_first .. owed_first + owed - 1 (mod STAGES)
                    const int items = g.tiles * g.splits;
                    unsigned long long t0 = 0;
                    auto settle = [&]() {              // the activations may be read now: pay what is owed
                        asm volatile("fence.proxy.async;" ::: "memory");
                        go = true;
                        for (int i = 0; i < owed; ++i) {
                            const int st = (owed_first + i) % STAGES;
                            tma_load_2d(smem_u32(smem + st * STAGE_BYTES) + P_BYTES, &g.map_x, owed_kb[st] * TILE_K, 0,
                                        full0 + 8 * st);
                        }
                        owed = 0;
                    };
                    auto stalled = [&]() {             // nothing can be issued: keep an eye on the clock
                        if (t0 == 0) t0 = global_ns();
                        if (ld_acquire(a.status) != 0 || global_ns() - t0 > WAIT_LIMIT_NS) {
                            atomicCAS(a.status, 0, 5);
                            ok = false;
                        }
                    };
                    for (int w = blockIdx.x; w < items && ok; w += grid) {
                        const int tile = w / g.splits, split = w - tile * g.splits;
                        const int kb0 = split * g.kb_per, kb1 = min(kb0 + g.kb_per, g.kb_total);
                        for (int kb = kb0; kb < kb1 && ok;) {
                            if (!go && *passed >= need) settle();
                            const bool free_now = first_pass || mbar_try(empty0 + 8 * stage, phase ^ 1);
                            if (!free_now || (!go && owed == STAGES)) {
                                stalled();
                                continue;
                            }
                            t0 = 0;
                            const uint32_t dst = smem_u32(smem + stage * STAGE_BYTES);
                            mbar_expect_tx(full0 + 8 * stage, STAGE_BYTES);
                            tma_load_2d(dst, &g.map_w, kb * TILE_K, tile * TILE_P, full0 + 8 * stage);
                            if (go) {
                                tma_load_2d(dst + P_BYTES, &g.map_x, kb * TILE_K, 0, full0 + 8 * stage);
                            } else {
                                owed_kb[stage] = kb;
                                ++owed;
                            }
                            if (++stage == STAGES) { stage = 0; phase ^= 1; first_pass = false; }
                            ++kb;
                        }
                    }
                    while (ok && !go) {                // do not enter the next product with debts
                        if (*passed >= need) settle();
                        else stalled();
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(TILE_P, BN);
            int stage = 0, it = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int l = 0; l < a.n_layers && ok; ++l) {
                const LayerArgs& L = a.layers[l];
                for (int ph = 0; ph < 4 && ok; ++ph) {
                    const GemmPhase& g = ph == 0 ? L.qkv : ph == 1 ? L.o : ph == 2 ? L.gu : L.down;
                    const int items = g.tiles * g.splits;
                    for (int w = blockIdx.x; w < items && ok; w += grid, ++it) {
                        const int tile = w / g.splits, split = w - tile * g.splits;
                        const int kb0 = split * g.kb_per, kb1 = min(kb0 + g.kb_per, g.kb_total);
                        const int ai = it & 1;
                        if (!(ok = mbar_wait(acce0 + 8 * ai, ((it >> 1) & 1) ^ 1, a.status, 2))) break;
                        tc_fence_after();
                        const uint32_t d_tmem = tmem_base + ai * BN;
                        for (int kb = kb0; kb < kb1; ++kb) {
                            if (!(ok = mbar_wait(full0 + 8 * stage, phase, a.status, 3))) break;
                            tc_fence_after();
                            const uint32_t pa = smem_u32(smem + stage * STAGE_BYTES);
                            const uint64_t da = smem_desc(pa), db = smem_desc(pa + P_BYTES);
#pragma unroll
                            for (int k = 0; k < TILE_K / UMMA_K; ++k)
                                tc_mma(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                            tc_commit(empty0 + 8 * stage);
                            if (++stage == STAGES) { stage = 0; phase ^= 1; }
                        }
                        if (ok) tc_commit(accf0 + 8 * ai);
                    }
                }
            }
        }
    } else {
        const int wt = threadIdx.x - 64;               // 0..127 among the workers
        const int quarter = warp & 3;
        const int i_local = quarter * 32 + lane;
        const int G = a.nq / a.nkv;
        const int row_tiles = (G + 15) / 16;
        int it = 0, g_no = 0;
        bool ok = true;
        fr_pdl_wait();
        if (a.trace != nullptr && blockIdx.x == 0 && wt == 0) a.trace[0] = global_ns();

        auto epilogue = [&](const GemmPhase& g) {
            Epi ep{g.out, g.bias, g.residual, g.n, a.rows, g.ldo, FR_BF16, g.bias_dtype, 1, g.act};
            const int items = g.tiles * g.splits;
            for (int w = blockIdx.x; w < items && ok; w += grid, ++it) {
                const int tile = w / g.splits, split = w - tile * g.splits;
                const int ai = it & 1;
                if (!(ok = mbar_wait(accf0 + 8 * ai, (it >> 1) & 1, a.status, 4))) break;
                tc_fence_after();
                const int gi = tile * TILE_P + i_local;
                uint32_t r[16];
                tc_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + ai * BN, r);
                tc_ld_wait();
                float v[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acce0 + 8 * ai);
                if (g.splits == 1) {
                    finish16(ep, gi, 0, v);
                } else {
                    float* part = a.gemm_scratch + (size_t)w * TILE_P * BN + (size_t)i_local * 16;
#pragma unroll
                    for (int j = 0; j < 4; ++j) ((float4*)part)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    __threadfence();
                    worker_sync();
                    if (wt == 0) flags[0] = atomicAdd(a.gemm_counters + tile, 1) == g.splits - 1;
                    worker_sync();
                    if (flags[0]) {
                        __threadfence();
                        const float* first = a.gemm_scratch + (size_t)tile * g.splits * TILE_P * BN + (size_t)i_local * 16;
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.f;
#pragma unroll 4
                        for (int s = 0; s < g.splits; ++s) {
                            const float4* src = (const float4*)(first + (size_t)s * TILE_P * BN);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float4 x = __ldcg(src + j);
                                v[4 * j] += x.x; v[4 * j + 1] += x.y; v[4 * j + 2] += x.z; v[4 * j + 3] += x.w;
                            }
                        }
                        finish16(ep, gi, 0, v);
                        if (wt == 0) a.gemm_counters[tile] = 0;
                    }
                    worker_sync();
                }
            }
        };

        for (int l = 0; l < a.n_layers && ok; ++l) {
            const LayerArgs& L = a.layers[l];
            for (int b = blockIdx.x; b < a.rows; b += grid)
                norm_row(a.x + (size_t)b * a.width, FrVec{L.norm1_w, L.norm1_dtype}, a.xn + (size_t)b * a.width, a.width,
                         L.eps1, wt, red);
            if (!(ok = grid_barrier(a, g_no++, wt, passed))) break;
            epilogue(L.qkv);
            if (!ok || !(ok = grid_barrier(a, g_no++, wt, passed))) break;
            {
                const int heads = a.nq + 2 * a.nkv;
                for (int i = blockIdx.x; i < a.rows * heads; i += grid) rope_head(a, L, i / heads, i % heads, HD, wt);
            }
            if (!(ok = grid_barrier(a, g_no++, wt, passed))) break;
            {
                const int S = a.attn_splits;
                const int items = a.rows * a.nkv * row_tiles * S;
                for (int i = blockIdx.x; i < items; i += grid) {
                    const int split = i % S, tile = (i / S) % row_tiles, kvh = (i / (S * row_tiles)) % a.nkv;
                    const int row = i / (S * row_tiles * a.nkv);
                    attention_item<HD>(a, L, row, kvh, tile, split, smem_attn, wt);
                }
            }
            if (!(ok = grid_barrier(a, g_no++, wt, passed))) break;
            epilogue(L.o);
            if (!ok || !(ok = grid_barrier(a, g_no++, wt, passed))) break;
            for (int b = blockIdx.x; b < a.rows; b += grid)
                norm_row(a.x + (size_t)b * a.width, FrVec{L.norm2_w, L.norm2_dtype}, a.xn + (size_t)b * a.width, a.width,
                         L.eps2, wt, red);
            if (!(ok = grid_barrier(a, g_no++, wt, passed))) break;
            epilogue(L.gu);
            if (!ok || !(ok = grid_barrier(a, g_no++, wt, passed))) break;
            epilogue(L.down);
            if (!ok || !(ok = grid_barrier(a, g_no++, wt, passed))) break;
        }
        // Leave the barrier slots as they were found: the last CTA out clears them.
        worker_sync();
        if (wt == 0) {
            __threadfence();
            if (atomicAdd(a.grid_bars + 2, 1) == grid - 1) {
                a.grid_bars[0] = 0;
                a.grid_bars[1] = 0;
                a.grid_bars[2] = 0;
                __threadfence();
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)ptr;
    }
    return fn;
}

int make_map(CUtensorMap* map, const void* base, int rows, int k, int ld, int box_rows) {
    EncodeTiled enc = encode_fn();
    if (enc == nullptr) FR_REFUSE("decode_layer: the driver does not offer cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)TILE_K, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) FR_REFUSE("decode_layer: cuTensorMapEncodeTiled failed with %d", (int)r);
    return FR_OK;
}

int fill_phase(GemmPhase* g, const void* w, int n, int k, const void* x, int rows, void* out, int ldo, const void* bias,
               int bias_dtype, const void* residual, int act, int ctas) {
    if (k % 8 || ((uintptr_t)w & 15) || ((uintptr_t)x & 15)) FR_REFUSE("decode_layer: k = %d or an operand is not 16-byte aligned", k);
    int rc = make_map(&g->map_w, w, n, k, k, TILE_P);
    if (rc) return rc;
    rc = make_map(&g->map_x, x, rows, k, k, BN);
    if (rc) return rc;
    g->out = out; g->bias = bias; g->residual = residual; g->bias_dtype = bias_dtype; g->n = n; g->ldo = ldo; g->act = act;
    g->tiles = (n + TILE_P - 1) / TILE_P;
    g->kb_total = (k + TILE_K - 1) / TILE_K;
    int splits = 1;
    if (g->tiles * 2 <= ctas) {
        splits = ctas / g->tiles;
        if (splits > g->kb_total / 4) splits = g->kb_total / 4;
        if (splits < 1) splits = 1;
    }
    g->kb_per = (g->kb_total + splits - 1) / splits;
    g->splits = (g->kb_total + g->kb_per - 1) / g->kb_per;
    return FR_OK;
}

template <int HD>
int launch(const StepArgs& a, int ctas, cudaStream_t stream) {
    constexpr int ATTN_BYTES = 16 * (HD * 2 + 16) + 4 * KEYS * (HD * 2 + 16);
    constexpr int smem = STAGES * STAGE_BYTES + ((ATTN_BYTES + 15) & ~15) + (2 * STAGES + 4) * 8 + 64 + 1024;
    static bool configured = false;
    if (!configured) {
        FR_CUDA(cudaFuncSetAttribute(decode_layers_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured = true;
    }
    // A cooperative launch: every CTA must be resident, because CTAs wait for one another at the grid barriers.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    FR_CUDA(cudaLaunchKernelEx(&cfg, decode_layers_kernel<HD>, a));
    FR_CHECK_LAUNCH("decode_layers");
    return FR_OK;
}

}  // namespace

FR_EXPORT int decode_layer_args_bytes() { return (int)sizeof(LayerArgs); }

FR_EXPORT int decode_layer_supports(int rows, int hd, int width, int inner) {
    return rows >= 1 && rows <= BN && (hd == 16 || hd == 32 || hd == 64 || hd == 128) && width % 8 == 0 && inner % 8 == 0;
}

// Fills one LayerArgs (host memory, `dst`) for a layer; all pointers are device pointers.
// w_qkv [(nq+2nkv) hd][width] with b_qkv; w_o [width][nq hd]; w_gu [2 inner][width] (rows alternate gate, up);
// w_d [width][inner].  x, xn [rows][width]; qkv [rows][(nq+2nkv) hd]; attn [rows][nq hd]; act [rows][inner].
FR_EXPORT int decode_layer_fill(void* dst, int rows, int width, int nq, int nkv, int hd, int inner, const void* w_qkv,
                                const void* b_qkv, int b_dtype, const void* w_o, const void* w_gu, const void* w_d,
                                const void* norm1_w, int norm1_dtype, float eps1, const void* norm2_w, int norm2_dtype,
                                float eps2, void* x, void* xn, void* qkv, void* attn, void* act, void* k_pool,
                                void* v_pool, const int* block_table, int table_width, int window,
                                const float* rope_denom, int rot, int ctas) {
    if (!decode_layer_supports(rows, hd, width, inner)) FR_REFUSE("decode_layer: %d rows / head size %d is not built", rows, hd);
    if (rot < 0 || rot > hd || (rot & 1)) FR_REFUSE("decode_layer: rotary size %d", rot);
    LayerArgs* L = (LayerArgs*)dst;
    const int qkv_n = (nq + 2 * nkv) * hd, qd = nq * hd;
    int rc = fill_phase(&L->qkv, w_qkv, qkv_n, width, xn, rows, qkv, qkv_n, b_qkv, b_dtype, nullptr, 0, ctas);
    if (rc) return rc;
    rc = fill_phase(&L->o, w_o, width, qd, attn, rows, x, width, nullptr, 0, x, 0, ctas);
    if (rc) return rc;
    rc = fill_phase(&L->gu, w_gu, 2 * inner, width, xn, rows, act, inner, nullptr, 0, nullptr, 1, ctas);
    if (rc) return rc;
    rc = fill_phase(&L->down, w_d, width, inner, act, rows, x, width, nullptr, 0, x, 0, ctas);
    if (rc) return rc;
    L->norm1_w = norm1_w; L->norm2_w = norm2_w; L->norm1_dtype = norm1_dtype; L->norm2_dtype = norm2_dtype;
    L->eps1 = eps1; L->eps2 = eps2; L->k_pool = (bf16*)k_pool; L->v_pool = (bf16*)v_pool; L->block_table = block_table;
    L->table_width = table_width; L->window = window; L->rope_denom = rope_denom; L->rot = rot;
    return FR_OK;
}

// Scratch that the kernel needs: out[0] floats of split-k partial tiles, out[1] tile counters, out[2] floats of
// attention partials, out[3] attention counters, for the layer described by `layer` (host LayerArgs).
FR_EXPORT int decode_layer_scratch(const void* layer, int rows, int nq, int nkv, int hd, int attn_splits, long long* out) {
    const LayerArgs* L = (const LayerArgs*)layer;
    long long floats = 0, counters = 0;
    const GemmPhase* ph[4] = {&L->qkv, &L->o, &L->gu, &L->down};
    for (int i = 0; i < 4; ++i) {
        if (ph[i]->splits > 1) {
            const long long f = (long long)ph[i]->tiles * ph[i]->splits * TILE_P * BN;
            floats = f > floats ? f : floats;
            counters = ph[i]->tiles > counters ? ph[i]->tiles : counters;
        }
    }
    out[0] = floats; out[1] = counters;
    out[2] = attn_splits > 1 ? (long long)rows * nq * attn_splits * (hd + 2) : 0;
    out[3] = (long long)rows * nkv * ((nq / nkv + 15) / 16);
    return FR_OK;
}

// Runs n_layers layers (device array `layers` of LayerArgs) on the rows' residual stream x, in place.
// grid_bars: 3 zeroed ints (left zeroed); counters zeroed (left zeroed); status: a device int; trace: null, or
// n_layers * 8 + 1 64-bit words that receive the times (ns) at which CTA 0 started and left each grid barrier.
FR_EXPORT int decode_layers_run(const void* layers, int n_layers, void* x, void* xn, void* qkv, void* attn,
                                const int* row_seq, const int* row_pos, float* gemm_scratch, int* gemm_counters,
                                float* attn_scratch, int* attn_counters, int attn_splits, int* grid_bars, int* status,
                                unsigned long long* trace, int rows, int width, int nq, int nkv, int hd, float scale,
                                int ctas, cudaStream_t stream) {
    if (n_layers <= 0) return FR_OK;
    if (((uintptr_t)layers & 63)) FR_REFUSE("decode_layer: the layer array must be 64-byte aligned");
    if (attn_splits < 1 || attn_splits > 64) FR_REFUSE("decode_layer: %d attention splits", attn_splits);
    StepArgs a;
    a.layers = (const LayerArgs*)layers; a.x = (bf16*)x; a.xn = (bf16*)xn; a.qkv = (bf16*)qkv; a.attn = (bf16*)attn;
    a.row_seq = row_seq; a.row_pos = row_pos; a.gemm_scratch = gemm_scratch; a.gemm_counters = gemm_counters;
    a.attn_scratch = attn_scratch; a.attn_counters = attn_counters; a.grid_bars = grid_bars; a.status = status;
    a.trace = trace;
    a.n_layers = n_layers; a.rows = rows; a.width = width; a.nq = nq; a.nkv = nkv; a.attn_splits = attn_splits;
    a.scale_log2 = scale * LOG2E;
    switch (hd) {
        case 16: return launch<16>(a, ctas, stream);
        case 32: return launch<32>(a, ctas, stream);
        case 64: return launch<64>(a, ctas, stream);
        case 128: return launch<128>(a, ctas, stream);
        default: FR_REFUSE("decode_layer: head size %d is not built", hd);
    }
}
