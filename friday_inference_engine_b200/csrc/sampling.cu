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
// A row is shared by the CTAs of one thread-block cluster (up to 8, each with a
// contiguous range of the vocabulary, 1024 threads each): one CTA alone reads a
// 150,000-entry row at a fraction of the memory bandwidth.  Every thread owns a
// contiguous piece of its CTA's range, so the running sum is taken in the order of
// the token ids; maxima and range totals cross the cluster through shared memory.
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

__device__ __forceinline__ bool better(float v, int i, float best, int best_i) {
    return v > best || (v == best && i < best_i);       // the first maximum wins
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, int ld, const float* __restrict__ temperature,
              const int* __restrict__ stream, const int* __restrict__ step, unsigned long long seed,
              const int* __restrict__ row_live, int* __restrict__ out, int ctas_per_row) {
    __shared__ float s_val[THREADS / 32];
    __shared__ int s_idx[THREADS / 32];
    __shared__ float s_scan[THREADS];
    __shared__ float s_best;       // this CTA's greatest finite logit, its first index, and its sum of exponentials:
    __shared__ float s_best_i;     // read by the other CTAs of the cluster (the index as a float's bits)
    __shared__ float s_total;
    fr_pdl_wait();
    fr_pdl_launch();
    const int C = ctas_per_row;
    const int row = blockIdx.x / C, rank = blockIdx.x - row * C;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // every CTA of a cluster takes the same path: the conditions below depend on the row only
    if (row_live != nullptr && row_live[row] < 0) {
        if (tid == 0 && rank == 0) out[row] = 0;
        return;
    }
    const float* x = logits + (size_t)row * ld;
    const int range = (vocab + C - 1) / C;
    const int r0 = min(rank * range, vocab), r1 = min(r0 + range, vocab);

    // Greatest finite logit and its first index: this CTA's range, then the cluster.
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = r0 + tid; i < r1; i += THREADS) {
        const float v = x[i];
        if (finite(v) && v > best) { best = v; best_i = i; }     // i ascends: the first maximum stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        best = s_val[lane]; best_i = s_idx[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
        }
        if (lane == 0) { s_best = best; s_best_i = __int_as_float(best_i); }
    }
    fr_cluster_sync();
    best = -INFINITY;
    best_i = 0x7fffffff;
    for (int r = 0; r < C; ++r) {
        const float ov = fr_cluster_load(&s_best, r);
        const int oi = __float_as_int(fr_cluster_load(&s_best_i, r));
        if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
    }
    const int greedy = best_i == 0x7fffffff ? -1 : best_i;
    const float t = temperature[row];
    if (!(t > 0.f) || greedy < 0) {
        if (tid == 0 && rank == 0) out[row] = greedy;
        fr_cluster_sync();                              // nobody leaves while its shared memory may still be read
        return;
    }

    // Sum of exp((x - max) / t) over this thread's contiguous piece of the CTA's range.
    const float inv_t = 1.0f / t, big = best;
    const int piece = (r1 - r0 + THREADS - 1) / THREADS;
    const int i0 = min(r0 + tid * piece, r1), i1 = min(i0 + piece, r1);
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
    if (tid == 0) s_total = s_scan[THREADS - 1];
    fr_cluster_sync();
    // The ranges' sums in rank order: what lies before this CTA's range, and the whole.
    float offset = 0.f, total = 0.f;
    for (int r = 0; r < C; ++r) {
        if (r == rank) offset = total;
        total += fr_cluster_load(&s_total, r);
    }
    const float target = uniform_for(seed, (uint32_t)stream[row], (uint32_t)step[row]) * total;
    const float before = offset + (tid > 0 ? s_scan[tid - 1] : 0.f);
    const float upto = offset + s_scan[tid];
    if (before <= target && target < upto) {            // exactly one thread of the cluster, if any
        float run = before;
        int pick = -1, last = -1;
        for (int i = i0; i < i1; ++i) {
            const float v = x[i];
            if (!finite(v)) continue;
            run += expf((v - big) * inv_t);
            last = i;
            if (run > target) { pick = i; break; }
        }
        out[row] = pick >= 0 ? pick : last;
    }
    if (rank == 0 && tid == 0 && !(target < total)) out[row] = greedy;     // rounding pushed the target past the sum
    fr_cluster_sync();
}

}  // namespace

// logits: [rows][ld] fp32, `vocab` of each row used.  temperature, stream, step: one
// per row.  row_live (may be null): a negative entry marks a padding row, which gets 0.
FR_EXPORT int sampling_sample(const float* logits, int rows, int vocab, int ld, const float* temperature,
                              const int* stream_ids, const int* steps, unsigned long long seed, const int* row_live,
                              int* out, cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    if (vocab <= 0) FR_REFUSE("sample: vocabulary of %d", vocab);
    // CTAs per row: one per 16,384 entries, up to the 8 of a portable cluster
    int per_row = (vocab + 16383) / 16384;
    per_row = per_row < 1 ? 1 : per_row > 8 ? 8 : per_row;
    FR_CUDA(fr_launch_cluster(sample_kernel, dim3(rows * per_row), dim3(THREADS), 0, stream, (unsigned)per_row, logits,
                              vocab, ld, temperature, stream_ids, steps, seed, row_live, out, per_row));
    FR_CHECK_LAUNCH("sample");
    return FR_OK;
}
