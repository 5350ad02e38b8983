// Merging the partial results of attention over split key ranges; shared by the CUDA-core
// and the tensor-core attention kernels.  A split leaves, per (row, head): its weighted
// values o (unnormalised), its maximum score m (natural-log units) and its sum l.
#pragma once
#include <math.h>

#include "common.cuh"

struct MergeArgs {
    const float* part;   // [rows * nq][splits][hd + 2]
    void* out;           // [rows][nq * hd]
    int rows, nq, hd, splits;
};

constexpr int FR_MERGE_PER_LANE = 8;   // head sizes up to 256

// o = sum_s o_s exp(m_s - M) / sum_s l_s exp(m_s - M), M = max_s m_s; a split that saw
// no key has l = 0 and m = -inf and drops out.
template <typename T>
__global__ void __launch_bounds__(128) attention_merge_kernel(MergeArgs p) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * 4 + warp;
    if (item >= p.rows * p.nq) return;
    const float* part = p.part + (size_t)item * p.splits * (p.hd + 2);
    float big = -INFINITY;
    for (int s = 0; s < p.splits; ++s) big = fmaxf(big, part[(size_t)s * (p.hd + 2) + p.hd]);
    float l = 0.f, acc[FR_MERGE_PER_LANE];
#pragma unroll
    for (int i = 0; i < FR_MERGE_PER_LANE; ++i) acc[i] = 0.f;
    for (int s = 0; s < p.splits; ++s) {
        const float* ps = part + (size_t)s * (p.hd + 2);
        const float ls = ps[p.hd + 1];
        if (!(ls > 0.f)) continue;
        const float f = expf(ps[p.hd] - big);
        l += ls * f;
#pragma unroll
        for (int i = 0; i < FR_MERGE_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < p.hd) acc[i] += ps[d] * f;
        }
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    T* o_row = (T*)p.out + (size_t)item * p.hd;
#pragma unroll
    for (int i = 0; i < FR_MERGE_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < p.hd) fr_store(o_row + d, acc[i] * inv);
    }
}

