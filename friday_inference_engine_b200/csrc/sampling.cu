// Choosing a token from a row of fp32 logits, on the device: only the chosen ids
// cross to the host.
//
// temperature == 0: the greatest logit, NaN and Inf skipped, the first maximum
// wins, as the reference's argmaxLogits (main.cpp:90-101).
// temperature > 0: p = softmax(logits / temperature) in fp32 and the first token
// whose running sum of p exceeds u.  u is the upper 24 bits of the first word of
// Philox-4x32-10 with counter (step, stream, 0, 0) and key (seed lo, seed hi): a
// sequence's draws depend on its own stream number and step only, never on its
// batch-mates.  The reference samples greedily only; this part is this library's.
//
// One block of 1024 threads per row; each thread owns a contiguous piece of the row
// so that the running sum is taken in the order of the token ids.
#include <math.h>

#include "common.cuh"

FR_EXPORT const char* sampling_last_error() { return fr_error_text; }

namespace {

constexpr int THREADS = 1024;

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t (&k)[2]) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k[0], n2 = hi0 ^ c[3] ^ k[1];
    c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
    k[0] += 0x9E3779B9u; k[1] += 0xBB67AE85u;
}

__device__ float uniform_for(unsigned long long seed, uint32_t stream, uint32_t step) {
    uint32_t c[4] = {step, stream, 0u, 0u};
    uint32_t k[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
#pragma unroll
    for (int r = 0; r < 10; ++r) philox_round(c, k);
    return (float)(c[0] >> 8) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ bool finite(float v) { return !(isnan(v) || isinf(v)); }

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, int ld, const float* __restrict__ temperature,
              const int* __restrict__ stream, const int* __restrict__ step, unsigned long long seed,
              const int* __restrict__ row_live, int* __restrict__ out) {
    __shared__ float s_val[THREADS / 32];
    __shared__ int s_idx[THREADS / 32];
    __shared__ float s_scan[THREADS];
    __shared__ float s_max;
    __shared__ int s_pick;
    fr_pdl_wait();
    fr_pdl_launch();
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (row_live != nullptr && row_live[row] < 0) {
        if (tid == 0) out[row] = 0;
        return;
    }
    const float* x = logits + (size_t)row * ld;

    // Greatest finite logit and its first index.
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = tid; i < vocab; i += THREADS) {
        const float v = x[i];
        if (finite(v) && v > best) { best = v; best_i = i; }     // i ascends: the first maximum stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        best = s_val[lane]; best_i = s_idx[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        if (lane == 0) { s_max = best; s_pick = best_i == 0x7fffffff ? -1 : best_i; }
    }
    __syncthreads();
    const float t = temperature[row];
    if (!(t > 0.f) || s_pick < 0) {
        if (tid == 0) out[row] = s_pick;
        return;
    }

    // Sum of exp((x - max) / t) over this thread's contiguous piece.
    const float inv_t = 1.0f / t, big = s_max;
    const int piece = (vocab + THREADS - 1) / THREADS;
    const int i0 = min(tid * piece, vocab), i1 = min(i0 + piece, vocab);
    float mine = 0.f;
    for (int i = i0; i < i1; ++i) {
        const float v = x[i];
        if (finite(v)) mine += expf((v - big) * inv_t);
    }
    s_scan[tid] = mine;
    __syncthreads();
    for (int o = 1; o < THREADS; o <<= 1) {             // inclusive scan, Hillis-Steele
        const float add = tid >= o ? s_scan[tid - o] : 0.f;
        __syncthreads();
        s_scan[tid] += add;
        __syncthreads();
    }
    const float total = s_scan[THREADS - 1];
    const float target = uniform_for(seed, (uint32_t)stream[row], (uint32_t)step[row]) * total;
    const float before = tid > 0 ? s_scan[tid - 1] : 0.f;
    const float upto = s_scan[tid];
    if (tid == 0) s_pick = -1;
    __syncthreads();
    if (before <= target && target < upto) {            // exactly one thread, if any
        float run = before;
        int pick = -1, last = -1;
        for (int i = i0; i < i1; ++i) {
            const float v = x[i];
            if (!finite(v)) continue;
            run += expf((v - big) * inv_t);
            last = i;
            if (run > target) { pick = i; break; }
        }
        s_pick = pick >= 0 ? pick : last;
    }
    __syncthreads();
    if (tid == 0) out[row] = s_pick >= 0 ? s_pick : best_i;   // rounding pushed the target past the sum
}

}  // namespace

// logits: [rows][ld] fp32, `vocab` of each row used.  temperature, stream, step: one
// per row.  row_live (may be null): a negative entry marks a padding row, which gets 0.
FR_EXPORT int sampling_sample(const float* logits, int rows, int vocab, int ld, const float* temperature,
                              const int* stream_ids, const int* steps, unsigned long long seed, const int* row_live,
                              int* out, cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    if (vocab <= 0) FR_REFUSE("sample: vocabulary of %d", vocab);
    FR_CUDA(fr_launch(sample_kernel, dim3(rows), dim3(THREADS), 0, stream, logits, vocab, ld, temperature, stream_ids,
                      steps, seed, row_live, out));
    FR_CHECK_LAUNCH("sample");
    return FR_OK;
}
