// Optional work at the two ends of the tensor-core product (gemm_tc_fused); a zeroed struct asks for none.
// The three parts exist so that a one-token step needs no separate kernels between its products: each of them
// would cost a few microseconds of launch and dependency latency for a few kilobytes of work.  The reference
// fuses the same neighbours the other way round, into its row-wise kernels (residual add with the norm:
// cuda_math_kernels.cu:323-361; rotation with the cache write: cuda_math_kernels.cu:363-404).
#pragma once

struct GemmFusion {
    // (1) RMSNorm of the input, finished here.  The input rows x are g (*) u, rounded to bf16, of rows u whose
    // sums of squares arrive as `in_parts` partial sums per row, in_ssq[part][row]; every row of the product is
    // multiplied by 1 / sqrt(sum / in_width + in_eps) before bias, activation and residual.
    const float* in_ssq;
    int in_parts;
    float in_width, in_eps;
    // (2) RMSNorm of the output, begun here (few rows, bf16 output, n a multiple of 128): norm_out [m][ldo]
    // receives norm_w (*) out, rounded, and out_ssq[n / 128][m] each 128-column tile's share of the rows' sums of
    // squares.  The product that reads norm_out finishes the norm through (1).
    const void* norm_w;
    void* norm_out;
    float* out_ssq;
    int norm_w_dtype;
    // (3) Rotary encoding and cache write (few rows, bf16 output): the output is [q heads | k heads | v heads] of
    // hd columns each, hd a divisor of 128.  Row r belongs to sequence row_seq[r] (negative: skipped) at position
    // row_pos[r]; with denom (rot / 2 fp32 denominators) the pairs (i, i + rot / 2) of every q and k head are
    // rotated by pos / denom[i]; with pools, k and v go to the cache row that `table` gives the position.
    const int* row_seq;
    const int* row_pos;
    const float* denom;
    void* k_pool;
    void* v_pool;
    const int* table;
    int rot, nq, nkv, hd, table_width, page;
    // (4) For measurements: trace[cta][16] receives %globaltimer at points of the CTA's life (0 kernel entry,
    // 1 set-up done, 2 weights requested, 3 predecessor finished, 4 first operands landed, 5 last product issued,
    // 6 last accumulator complete, 7 last tile done; of a CTA that sums a tile's partial tiles: 8 it knows, 9 fence
    // passed, 10 partial tiles summed, 11 tile staged, 12 tile written).
    unsigned long long* trace;
};
