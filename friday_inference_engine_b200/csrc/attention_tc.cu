// Causal grouped-query attention for prompts on the 5th-generation tensor cores (sm_100a): both products of
// flash attention are tcgen05.mma with their results in tensor memory.
//
// A CTA owns up to 128 rows of one sequence and kv head; row r stands for (token r / G, group head r % G),
// G = heads / kv heads, so a block of keys and values is read once for all heads that share it (as the reference's
// R = tq*G + g rows: attention_kernels.cu:493-499).  A block of 64 keys is one page of the cache; even and odd blocks
// alternate between two stages of everything a block needs (K, V, the columns of S, the barriers).
//
//   warp 0      TMA producer: the queries (a 4-d box [64 dims][G heads][1][T tokens] per 64-dim slice lands as
//               rows t*G + g, 128-byte swizzle), then the K page of the block after and the V page of this one.  A
//               stage of K is free again once its scores are done, one of V after the second product.  A page that
//               the block does not need, or that the table does not name, is loaded from beyond the pool's last row,
//               which fills zeros.
//   warp 1      allocates tensor memory (256 columns: S of even blocks, S of odd blocks, O); one lane issues
//               S = Q K^T (M = 128 rows, N = 64 keys, both operands K-major from shared memory) two blocks ahead of
//               O += P V (A = P from tensor memory, where it lies over the first half of its S's columns; B = V as
//               it lies in the cache, [keys][dims] = MN-major): the scores of block i + 1 are ready when the rows
//               have finished block i, and the tensor core works on one block's products while the rows
//               exponentiate the other's.
//   warps 2-5   one thread per row (its TMEM lane): reads its 64 scores from tensor memory, takes maximum and
//               exponentials, keeps the running maximum and sum, and writes P (bf16, two to a column) back into
//               tensor memory.  The maximum that P is taken against only moves when a row's true maximum has grown
//               by more than 8 (in log2 units; P then stays below 2^8 and the sums remain exact for that reference);
//               only then is O rescaled, in tensor memory.  At the end the row's O is divided by its sum.
//
// Neither P nor O ever leaves tensor memory before the output is written.  A CTA needs 97 KB of shared memory and
// half the tensor memory, so two share an SM.
// Scores, softmax and sums are fp32; P is rounded to bf16 for the second product, as the mma.sync kernel does.
// Rows of V past the last key that any row of the CTA may see are zeroed in shared memory before the product (their
// P is zero, but zero times a stale NaN is not); stale K only reaches scores that the mask replaces.  Long tiles (late
// tokens) are launched first.  Every wait on an mbarrier is bounded (two seconds), then a code goes to `status` and
// all roles leave their loops.
//
// Head sizes: multiples of 16 up to 128.  One-token steps keep the mma.sync kernel (attention_mma.cu), whose rows
// of a CTA share a token.
#include <cuda.h>
#include <math.h>

#include <type_traits>

#include "common.cuh"
#include "tc_common.cuh"

FR_EXPORT const char* attention_tc_last_error() { return fr_error_text; }

namespace {

using namespace tc;
typedef __nv_bfloat16 bf16;
constexpr int THREADS = 192;
constexpr int ROWS = 128;                 // rows of a CTA = M of the instruction
constexpr int KEYS = 64;                  // keys of a block = one cache page
constexpr int PAGE = 64;
constexpr int SLICE = ROWS * 128;         // bytes of 128 rows of 64 bf16 (one 128-byte swizzle row each)
constexpr int KSLICE = KEYS * 128;        // bytes of a block's keys (or values), 64 dims of them
constexpr int KV_STAGE = 2 * KSLICE;      // a block's keys (or values): two slices of 64 dims
constexpr int TMEM_COLS = 256;           // S of even blocks | S of odd blocks (P over the first half of each) | O
constexpr float LOG2E = 1.4426950408889634f;

struct TcArgs {
    bf16* out;                // [rows][nq * hd]
    const int* block_table;   // [seqs][table_width]
    const int* seq_start;     // first row of each sequence
    const int* seq_qlen;      // rows (tokens) of each sequence in this step
    const int* seq_pos0;      // position of its first row
    const int* seq_live;      // may be null; < 0 at seq_start[s]: the sequence has ended
    int* status;
    int table_width, nq, nkv, hd, window, pool_rows, n_seqs;
    float scale_log2;         // softmax scale times log2(e)
    unsigned long long* trace;   // for measurements (may be null): [cta][8] sums of time (ns) that row 0's thread spent
                                 // waiting for S, reading it, writing P, rescaling O, waiting for the last product;
                                 // then blocks, total time, start
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
        : "memory");
}
// Descriptor of an MN-major operand (the contiguous dimension is N): 8 consecutive k form a 1024-byte swizzle atom
// of 64 n; `sbo` is the distance between atoms along k, `lbo` between atoms along n.
__device__ __forceinline__ uint64_t smem_desc_mn(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// 32 consecutive columns of this thread's TMEM lane
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, "
        "%24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, "
        "%25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tc_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 2^x by the special-function unit alone: exp2f() adds a range fix for results below 2^-126, which a probability
// that is rounded to bf16 and summed in fp32 has no use for (they become 0 here).
__device__ __forceinline__ float exp2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// 16 consecutive columns of this thread's TMEM lane, written
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand lies in tensor memory (lane = row, two bf16 per 32-bit column)
__device__ __forceinline__ void tc_mma_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__global__ void __launch_bounds__(THREADS, 2)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const TcArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* s_q = smem;                              // [2 slices][128 rows][128 B]
    uint8_t* s_k = s_q + 2 * SLICE;                   // [2 stages][2 slices][64 keys][128 B]
    uint8_t* s_v = s_k + 2 * KV_STAGE;                // [2 stages][2 slices of 64 dims][64 keys][128 B]
    uint64_t* bars = (uint64_t*)(s_v + 2 * KV_STAGE);
    // bars: q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], pv_done[2]
    uint32_t* tmem_slot = (uint32_t*)(bars + 15);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t q_full = smem_u32(bars), k_full = smem_u32(bars + 1), k_empty = smem_u32(bars + 3);
    const uint32_t v_full = smem_u32(bars + 5), v_empty = smem_u32(bars + 7);
    const uint32_t s_full = smem_u32(bars + 9), p_full = smem_u32(bars + 11), pv_done = smem_u32(bars + 13);
    // the barrier of stage b of a pair lies 8 bytes after that of stage 0

    // The CTA's rows and its range of key blocks.  The step's geometry is final before the step's first kernel
    // starts (common.cuh), so it is read ahead of the wait.
    // The grid is one line of CTAs, long tiles (late tokens) first over all sequences and kv heads: CTAs start in the
    // order of their index, and the longest tile bounds the launch (one prompt of 2,048 tokens: 71 us with the kv
    // heads as a grid dimension of their own, whose last head's long tiles started after the first heads' short
    // ones; 53 us in this order).  x = (tile rank * kv heads + kv head) * sequences + sequence.
    const int seq = blockIdx.x % p.n_seqs;
    const int kvh = (blockIdx.x / p.n_seqs) % p.nkv;
    const int n_tiles = gridDim.x / (p.n_seqs * p.nkv);
    const int tile = n_tiles - 1 - blockIdx.x / (p.n_seqs * p.nkv);
    const int G = p.nq / p.nkv, T = ROWS / G;         // T tokens of G heads each fill the tile's rows
    const int q_len = p.seq_qlen[seq], q_start = p.seq_start[seq], pos0 = p.seq_pos0[seq];
    const int t0 = tile * T;
    if (t0 >= q_len) return;
    if (p.seq_live != nullptr && p.seq_live[q_start] < 0) return;     // an ended sequence's rows are not written
    const int t_end = min(t0 + T, q_len);             // tokens t0 .. t_end-1
    const int pos_hi = pos0 + t_end - 1;              // the farthest key any row of the CTA may see
    const int lo_min = p.window > 0 ? max(0, pos0 + t0 - p.window + 1) : 0;
    const int kb_begin = lo_min / KEYS, kb_end = pos_hi / KEYS;       // inclusive
    const int n_blocks = kb_end - kb_begin + 1;
    const int slices = (p.hd + 63) / 64;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(k_full + 8 * b, 1);
            mbar_init(k_empty + 8 * b, 1);
            mbar_init(v_full + 8 * b, 1);
            mbar_init(v_empty + 8 * b, 1);
            mbar_init(s_full + 8 * b, 1);
            mbar_init(p_full + 8 * b, 128);
            mbar_init(pv_done + 8 * b, 1);
        }
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
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 2 * KEYS;      // columns: S0 | S1 (P over each one's first half) | O
    fr_pdl_wait();
    if (threadIdx.x == 0) fr_pdl_launch();

    // Block i of the CTA uses stage i & 1 of K, V and S; its barriers are in their (i >> 1)-th use.
    if (warp == 0) {
        if (elect_one()) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
            mbar_expect_tx(q_full, (uint32_t)slices * 64 * G * T * 2);
            for (int s = 0; s < slices; ++s)
                tma_load_4d(smem_u32(s_q + s * SLICE), &map_q, s * 64, 0, kvh, q_start + t0, q_full);
            const int* table = p.block_table + (size_t)seq * p.table_width;
            // the pool row of block i's page; a page that the table does not name is loaded from beyond the pool's last
            // row, which fills zeros
            auto page_row = [&](int i) {
                const int lp = kb_begin + i;
                if (lp * PAGE <= pos_hi && lp < p.table_width) {
                    const int page = table[lp];
                    if (page >= 0) return page * PAGE;
                }
                return p.pool_rows;
            };
            // a stage is free again when the product that read it is done: K after the scores, V after the second product
            auto load = [&](int i, const CUtensorMap* map, uint8_t* ring, uint32_t full, uint32_t empty) {
                const int b = i & 1, par = (i >> 1) & 1;
                if (!mbar_wait(empty + 8 * b, par ^ 1, p.status, 1)) return false;
                mbar_expect_tx(full + 8 * b, (uint32_t)slices * KSLICE);
                const int row = page_row(i);
                for (int s = 0; s < slices; ++s)
                    tma_load_3d(smem_u32(ring) + (uint32_t)(b * KV_STAGE + s * KSLICE), map, s * 64, kvh, row, full + 8 * b);
                return true;
            };
            // in the order in which the products want them: K of the block after, then V of this one
            bool ok = load(0, &map_k, s_k, k_full, k_empty);
            for (int i = 0; i < n_blocks && ok; ++i) {
                if (i + 1 < n_blocks) ok = load(i + 1, &map_k, s_k, k_full, k_empty);
                if (ok) ok = load(i, &map_v, s_v, v_full, v_empty);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            const uint32_t idesc_qk = instr_desc(ROWS, KEYS);
            const uint32_t idesc_pv = instr_desc(ROWS, p.hd) | (1u << 16);   // B is MN-major
            const int k_steps = p.hd / 16;                                   // of the first product
            bool ok = mbar_wait(q_full, 0, p.status, 2);
            unsigned long long m_spent[5] = {0, 0, 0, 0, 0}, m_mark = p.trace != nullptr ? global_ns() : 0;
            auto mlap = [&](int which) {
                if (p.trace != nullptr) {
                    const unsigned long long now = global_ns();
                    m_spent[which] += now - m_mark;
                    m_mark = now;
                }
            };
            // S[i & 1] = Q K_i^T.  The tensor core takes its instructions in order, so the columns of S[i & 1] (and P
            // over them) are free: the product P V of block i - 2 was issued earlier.
            auto scores = [&](int i) {
                const int b = i & 1, par = (i >> 1) & 1;
                if (!mbar_wait(k_full + 8 * b, par, p.status, 3)) return false;
                mlap(0);
                tc_fence_after();
                for (int ks = 0; ks < k_steps; ++ks) {
                    const int s = ks >> 2, k = ks & 3;
                    const uint64_t da = smem_desc(smem_u32(s_q + s * SLICE)) + 2 * k;
                    const uint64_t db = smem_desc(smem_u32(s_k + b * KV_STAGE + s * KSLICE)) + 2 * k;
                    tc_mma(tmem_s + b * KEYS, da, db, idesc_qk, ks > 0 ? 1u : 0u);
                }
                tc_commit(s_full + 8 * b);
                tc_commit(k_empty + 8 * b);
                mlap(1);
                return true;
            };
            // The scores run two blocks ahead of the second product: while the rows of block i exponentiate, the
            // scores of block i + 1 are done or under way.
            if (ok) ok = scores(0);
            if (ok && n_blocks > 1) ok = scores(1);
            for (int i = 0; i < n_blocks && ok; ++i) {
                const int b = i & 1, par = (i >> 1) & 1;
                if (!(ok = mbar_wait(v_full + 8 * b, par, p.status, 3))) break;
                mlap(2);
                if (!(ok = mbar_wait(p_full + 8 * b, par, p.status, 4))) break;
                mlap(3);
                tc_fence_after();
                // O += P V over the keys of this block that some row may see, in steps of 16; P from tensor memory
                const int keys_here = min(KEYS, pos_hi - (kb_begin + i) * KEYS + 1);
                const int pv_steps = (keys_here + 15) / 16;
                for (int ks = 0; ks < pv_steps; ++ks) {
                    const uint64_t db = smem_desc_mn(smem_u32(s_v) + b * KV_STAGE + ks * 16 * 128, KSLICE, 1024);
                    tc_mma_ta(tmem_o, tmem_s + b * KEYS + 8 * ks, db, idesc_pv, (i > 0 || ks > 0) ? 1u : 0u);
                }
                tc_commit(pv_done + 8 * b);
                tc_commit(v_empty + 8 * b);
                mlap(4);
                if (i + 2 < n_blocks) ok = scores(i + 2);
            }
            if (p.trace != nullptr) {
                unsigned long long* at = p.trace + (size_t)blockIdx.x * 16 + 8;
                for (int k = 0; k < 5; ++k) at[k] = m_spent[k];
            }
        }
    } else {
        const int quarter = warp & 3;                      // TMEM lanes this warp may read: 32*quarter ..
        const int r = quarter * 32 + lane;                 // this thread's row of the tile
        const int t = r / G, g = r - t * G;
        const bool valid = r < T * G && t0 + t < q_len;
        const int pos_r = valid ? pos0 + t0 + t : -1;      // -1: every key is masked
        const int lo_r = (valid && p.window > 0) ? max(0, pos_r - p.window + 1) : 0;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        float m_run = -INFINITY, l_run = 0.f;              // the maximum that P is taken against, and the sum of P
        bool ok = true;
        unsigned long long spent[5] = {0, 0, 0, 0, 0};
        const bool tracing = p.trace != nullptr && r == 0;
        unsigned long long t_mark = tracing ? global_ns() : 0, t_begin = t_mark;
        auto lap = [&](int which) {
            if (tracing) {
                const unsigned long long now = global_ns();
                spent[which] += now - t_mark;
                t_mark = now;
            }
        };
        for (int i = 0; i < n_blocks && ok; ++i) {
            const int b = i & 1, par = (i >> 1) & 1;
            const int kb = kb_begin + i;
            const int j0 = kb * KEYS;
            if (!(ok = mbar_wait(s_full + 8 * b, par, p.status, 6))) break;
            tc_fence_after();
            lap(0);
            // The row's 64 scores are read from tensor memory once and stay in registers for both passes.  Masked and
            // unmasked blocks have code of their own; most blocks need no mask (the choice must be the same for a whole
            // warp: loads from and stores to tensor memory are warp-wide instructions).
            const uint32_t s_addr = tmem_s + b * KEYS + lane_addr;
            // (Rows of the tile that stand for no token ask for no mask: what they compute stays in their own lanes of
            // tensor memory and is never written.  With them in the condition the warp of the tile's last rows, two of
            // which are such rows when 7 heads share a kv head, took the masked form in every block, 2.5 times as long
            // as the others.)
            const bool need_mask = __any_sync(0xffffffffu, j0 + KEYS - 1 > pos0 + t0 ||
                                                               (p.window > 0 && j0 < pos_hi - p.window + 1));
            uint32_t raw[KEYS];
            {
                uint32_t (&lo32)[32] = *reinterpret_cast<uint32_t (*)[32]>(&raw[0]);
                uint32_t (&hi32)[32] = *reinterpret_cast<uint32_t (*)[32]>(&raw[32]);
                tc_ld32(s_addr, lo32);
                tc_ld32(s_addr + 32, hi32);
                tc_ld_wait();
            }
            const int hi = pos_r - j0, lo = lo_r - j0;     // columns hi < j or j < lo are masked
            // The maximum of the raw scores in four strands (one strand of dependent comparisons would be paid in full:
            // a scheduler has few such warps to choose from); the positive scale is applied to the result.
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (need_mask) {
#pragma unroll
                for (int j = 0; j < KEYS; ++j) {
                    if (j > hi || j < lo) raw[j] = 0xff800000u;      // -inf
                    mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(raw[j]));
                }
            } else {
#pragma unroll
                for (int j = 0; j < KEYS; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(raw[j]));
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
            lap(1);
            // The reference maximum moves only when the true one has grown by more than 8; O is rescaled then.
            // tcgen05.ld and .st are warp-wide, so a warp rescales if any of its rows must.
            const bool grow = mx > m_run + 8.f;            // also the first finite maximum (m_run = -inf)
            if (__any_sync(0xffffffffu, grow)) {
                const float alpha = grow ? exp2f(m_run - mx) : 1.f;      // 0 for a row that had seen no key
                if (grow) {
                    m_run = mx;
                    l_run *= alpha;
                }
                if (i > 0) {
                    // every product into O so far must be done.  (The scores of this block were issued after the second
                    // product of block i - 2, so that one is done: a wait for a phase's parity is unambiguous only if
                    // the barrier is at most one phase behind, which is why the blocks alternate between two barriers.)
                    if (!(ok = mbar_wait(pv_done + 8 * (b ^ 1), ((i - 1) >> 1) & 1, p.status, 8))) break;
                    tc_fence_after();
#pragma unroll 1
                    for (int c = 0; c < 8; ++c) {
                        if (c * 16 < p.hd) {
                            uint32_t o16[16];
                            tc_ld16(tmem_o + lane_addr + c * 16, o16);
                            tc_ld_wait();
#pragma unroll
                            for (int j = 0; j < 16; ++j) o16[j] = __float_as_uint(__uint_as_float(o16[j]) * alpha);
                            tc_st16(tmem_o + lane_addr + c * 16, o16);
                        }
                    }
                    tc_st_wait();
                }
            }
            lap(3);
            // Exponentials; P (bf16, two to a column) goes over the first half of the columns of S.  A masked score is
            // -inf and stays so; a row that has seen no key takes its exponentials against 0.
            const float neg_m = m_run == -INFINITY ? 0.f : -m_run;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};            // four strands, for the same reason
            uint32_t packed[KEYS / 2];
#pragma unroll
            for (int j = 0; j < KEYS; j += 2) {
                const float e0 = exp2_fast(fmaf(__uint_as_float(raw[j]), p.scale_log2, neg_m));
                const float e1 = exp2_fast(fmaf(__uint_as_float(raw[j + 1]), p.scale_log2, neg_m));
                sum4[j & 2] += e0;
                sum4[(j & 2) + 1] += e1;
                packed[j >> 1] = pack2(e0, e1);
            }
            tc_st32(s_addr, packed);
            tc_st_wait();
            l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            if (kb == kb_end) {
                // keys past the last one that any row may see: their V rows may hold anything; zero them
                const int key = j0 + r;
                if (r < KEYS && key > pos_hi) {
                    if (!(ok = mbar_wait(v_full + 8 * b, par, p.status, 7))) break;
                    for (int s = 0; s < slices; ++s) {
                        uint4* line = (uint4*)(s_v + b * KV_STAGE + s * KSLICE + r * 128);
#pragma unroll
                        for (int q = 0; q < 8; ++q) line[q] = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            tc_fence_before();
            mbar_arrive(p_full + 8 * b);
            lap(2);
        }
        // the last product; then the row's output
        if (ok) ok = mbar_wait(pv_done + 8 * ((n_blocks - 1) & 1), ((n_blocks - 1) >> 1) & 1, p.status, 8);
        tc_fence_after();
        lap(4);
        if (ok) {
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            bf16* dst = p.out + ((size_t)(q_start + t0 + t) * p.nq + (size_t)kvh * G + g) * p.hd;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                if (c * 32 < p.hd) {                                   // uniform: the load is warp-wide
                    uint32_t o32[32];
                    tc_ld32(tmem_o + lane_addr + c * 32, o32);
                    tc_ld_wait();
                    if (valid) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            if (c * 32 + q * 8 < p.hd) {
                                float x[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(o32[q * 8 + j]) * inv;
                                *(uint4*)(dst + c * 32 + q * 8) =
                                    make_uint4(pack2(x[0], x[1]), pack2(x[2], x[3]), pack2(x[4], x[5]), pack2(x[6], x[7]));
                            }
                        }
                    }
                }
            }
        }
        if (tracing) {
            unsigned long long* at = p.trace + (size_t)blockIdx.x * 16;
            for (int k = 0; k < 5; ++k) at[k] = spent[k];
            at[5] = (unsigned long long)n_blocks;
            at[6] = global_ns() - t_begin;
            at[7] = t_begin;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ two row tiles per CTA
// The same attention with one CTA per SM that owns two consecutive row tiles of a sequence and kv head, blocks of 128
// keys (two pages), and the whole tensor memory: per tile 128 columns of S (P over the first 64) and 128 of O.  The
// tiles take turns on the tensor core: while the rows of one tile exponentiate, the core runs the other tile's
// O += P V and its next S = Q K^T, so neither waits for the other's softmax; a block of keys and values is loaded
// once for both tiles, and S = Q K^T has N = 128 (the operands' traffic from shared memory per product is half that
// of N = 64).  S has one stage per tile: a tile's next scores are issued right behind its second product, and the
// tensor core runs its instructions in order.
//
//   warp 0      TMA: both tiles' queries, then K of the block after and V of this one (two stages each)
//   warp 1      tensor memory (512 columns); one lane issues, per block, for tile 0 and then tile 1:
//               O += P V of this block, S = Q K^T of the next
//   warps 2-5   the rows of tile 0, warps 6-9 the rows of tile 1: one thread per row, as in the kernel above
constexpr int THREADS2 = 320;
constexpr int KEYS2 = 128;
constexpr int KSLICE2 = KEYS2 * 128;      // a block's keys (or values), 64 dims of them
constexpr int KV_STAGE2 = 2 * KSLICE2;
constexpr int SMEM_BYTES2 = 4 * SLICE + 4 * KV_STAGE2 + 1024 + 256;

__global__ void __launch_bounds__(THREADS2, 1)
attention_tc_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const TcArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* s_q = smem;                              // [2 tiles][2 slices][128 rows][128 B]
    uint8_t* s_k = s_q + 4 * SLICE;                   // [2 stages][2 slices][128 keys][128 B]
    uint8_t* s_v = s_k + 2 * KV_STAGE2;               // [2 stages][2 slices of 64 dims][128 keys][128 B]
    uint64_t* bars = (uint64_t*)(s_v + 2 * KV_STAGE2);
    // bars: q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2 tiles], p_full[2 tiles], o_done
    uint32_t* tmem_slot = (uint32_t*)(bars + 14);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t q_full = smem_u32(bars), k_full = smem_u32(bars + 1), k_empty = smem_u32(bars + 3);
    const uint32_t v_full = smem_u32(bars + 5), v_empty = smem_u32(bars + 7);
    const uint32_t s_full = smem_u32(bars + 9), p_full = smem_u32(bars + 11), o_done = smem_u32(bars + 13);

    // x = (pair rank * kv heads + kv head) * sequences + sequence, long pairs (late tokens) first
    const int seq = blockIdx.x % p.n_seqs;
    const int kvh = (blockIdx.x / p.n_seqs) % p.nkv;
    const int n_pairs = gridDim.x / (p.n_seqs * p.nkv);
    const int pair = n_pairs - 1 - blockIdx.x / (p.n_seqs * p.nkv);
    const int G = p.nq / p.nkv, T = ROWS / G;
    const int q_len = p.seq_qlen[seq], q_start = p.seq_start[seq], pos0 = p.seq_pos0[seq];
    if (2 * pair * T >= q_len) return;
    if (p.seq_live != nullptr && p.seq_live[q_start] < 0) return;
    // Per tile: its tokens, the farthest key any of its rows may see, and its blocks of 128 keys (inclusive).  The
    // second tile may not exist; its range never begins or ends before the first one's.
    int t0[2], pos_hi[2], kb0[2], kb1[2];
    bool active[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        t0[x] = (2 * pair + x) * T;
        active[x] = t0[x] < q_len;
        const int t_end = min(t0[x] + T, q_len);
        pos_hi[x] = pos0 + t_end - 1;
        const int lo_min = p.window > 0 ? max(0, pos0 + t0[x] - p.window + 1) : 0;
        kb0[x] = lo_min / KEYS2;
        kb1[x] = pos_hi[x] / KEYS2;
    }
    const int ub0 = kb0[0], ub1 = active[1] ? kb1[1] : kb1[0];
    const int n_blocks = ub1 - ub0 + 1;
    const int pos_hi_u = active[1] ? pos_hi[1] : pos_hi[0];
    const int slices = (p.hd + 63) / 64;
    auto part = [&](int x, int i) { return active[x] && ub0 + i >= kb0[x] && ub0 + i <= kb1[x]; };

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(k_full + 8 * b, 1);
            mbar_init(k_empty + 8 * b, 1);
            mbar_init(v_full + 8 * b, 1);
            mbar_init(v_empty + 8 * b, 1);
            mbar_init(s_full + 8 * b, 1);
            mbar_init(p_full + 8 * b, 128);
        }
        mbar_init(o_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;            // columns of tile x: S at 256 x (P over its first 64), O at 256 x + 128
    fr_pdl_wait();
    if (threadIdx.x == 0) fr_pdl_launch();

    // Block i of the CTA uses stage i & 1 of K and V, in their (i >> 1)-th use; a tile's barriers count its own blocks.
    if (warp == 0) {
        if (elect_one()) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
            mbar_expect_tx(q_full, (uint32_t)((active[1] ? 2 : 1) * slices * 64 * G * T * 2));
            for (int x = 0; x < 2; ++x)
                if (active[x])
                    for (int s = 0; s < slices; ++s)
                        tma_load_4d(smem_u32(s_q + (2 * x + s) * SLICE), &map_q, s * 64, 0, kvh, q_start + t0[x], q_full);
            const int* table = p.block_table + (size_t)seq * p.table_width;
            auto page_row = [&](int lp) {              // lp: the page's number in the sequence
                if (lp * PAGE <= pos_hi_u && lp < p.table_width) {
                    const int page = table[lp];
                    if (page >= 0) return page * PAGE;
                }
                return p.pool_rows;                    // beyond the pool: zeros
            };
            auto load = [&](int i, const CUtensorMap* map, uint8_t* ring, uint32_t full, uint32_t empty) {
                const int b = i & 1, par = (i >> 1) & 1;
                if (!mbar_wait(empty + 8 * b, par ^ 1, p.status, 1)) return false;
                mbar_expect_tx(full + 8 * b, (uint32_t)(2 * slices * KSLICE));
                for (int pg = 0; pg < 2; ++pg) {
                    const int row = page_row(2 * (ub0 + i) + pg);
                    for (int s = 0; s < slices; ++s)
                        tma_load_3d(smem_u32(ring) + (uint32_t)(b * KV_STAGE2 + s * KSLICE2 + pg * KSLICE), map, s * 64, kvh, row,
                                    full + 8 * b);
                }
                return true;
            };
            bool ok = load(0, &map_k, s_k, k_full, k_empty);
            for (int i = 0; i < n_blocks && ok; ++i) {
                if (i + 1 < n_blocks) ok = load(i + 1, &map_k, s_k, k_full, k_empty);
                if (ok) ok = load(i, &map_v, s_v, v_full, v_empty);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            const uint32_t idesc_qk = instr_desc(ROWS, KEYS2);
            const uint32_t idesc_pv = instr_desc(ROWS, p.hd) | (1u << 16);   // B is MN-major
            const int k_steps = p.hd / 16;
            bool ok = mbar_wait(q_full, 0, p.status, 2);
            int done[2] = {0, 0};                      // blocks whose second product a tile has issued
            unsigned long long m_spent[5] = {0, 0, 0, 0, 0}, m_mark = p.trace != nullptr ? global_ns() : 0;
            auto mlap = [&](int which) {
                if (p.trace != nullptr) {
                    const unsigned long long now = global_ns();
                    m_spent[which] += now - m_mark;
                    m_mark = now;
                }
            };
            // One thread issues every product, and a lone thread runs one dependent instruction every four or five
            // cycles: what an instruction costs to prepare decides whether the tensor core is kept busy (a product of
            // N = 128 takes it 64 cycles).  So the descriptors are made once and only stepped in the loops below.  (A
            // descriptor's low bits are the address in units of 16 bytes; offsets that stay inside the operand's buffer
            // never carry out of them.)
            const uint64_t dq0 = smem_desc(smem_u32(s_q)), dk0 = smem_desc(smem_u32(s_k));
            const uint64_t dv0 = smem_desc_mn(smem_u32(s_v), KSLICE2, 1024);
            auto scores = [&](int x, int i) {
                const int b = i & 1, par = (i >> 1) & 1;
                if (!mbar_wait(k_full + 8 * b, par, p.status, 3)) return false;
                mlap(0);
                tc_fence_after();
                uint64_t da = dq0 + (uint64_t)(x * (2 * SLICE >> 4)), db = dk0 + (uint64_t)(b * (KV_STAGE2 >> 4));
                const uint32_t d = tmem_base + 256 * x;
                for (int ks = 0; ks < k_steps; ++ks) {
                    tc_mma(d, da, db, idesc_qk, ks > 0 ? 1u : 0u);
                    // 32 bytes on in the 128-byte row; after four of them the next slice of 64 dims
                    da += (ks & 3) == 3 ? (uint64_t)((SLICE >> 4) - 6) : 2ull;
                    db += (ks & 3) == 3 ? (uint64_t)((KSLICE2 >> 4) - 6) : 2ull;
                }
                tc_commit(s_full + 8 * x);
                mlap(1);
                return true;
            };
            auto second = [&](int x, int i) {
                const int b = i & 1, par = (i >> 1) & 1;
                if (!mbar_wait(v_full + 8 * b, par, p.status, 3)) return false;
                mlap(2);
                if (!mbar_wait(p_full + 8 * x, done[x] & 1, p.status, 4)) return false;
                mlap(3);
                tc_fence_after();
                const int keys_here = min(KEYS2, pos_hi[x] - (ub0 + i) * KEYS2 + 1);
                const int pv_steps = (keys_here + 15) / 16;
                uint64_t db = dv0 + (uint64_t)(b * (KV_STAGE2 >> 4));
                const uint32_t d = tmem_base + 256 * x + 128;
                uint32_t pa = tmem_base + 256 * x;
                uint32_t keep = done[x] > 0 ? 1u : 0u;
                for (int ks = 0; ks < pv_steps; ++ks) {
                    tc_mma_ta(d, pa, db, idesc_pv, keep);
                    keep = 1u;
                    pa += 8;                               // 16 keys of P: 8 columns
                    db += (uint64_t)(16 * 128 >> 4);       // 16 keys of V
                }
                ++done[x];
                mlap(4);
                return true;
            };
            for (int x = 0; x < 2 && ok; ++x)
                if (part(x, 0)) ok = scores(x, 0);
            if (ok) tc_commit(k_empty);
            for (int i = 0; i < n_blocks && ok; ++i) {
                for (int x = 0; x < 2 && ok; ++x) {
                    if (part(x, i)) ok = second(x, i);
                    if (ok && i + 1 < n_blocks && part(x, i + 1)) ok = scores(x, i + 1);
                }
                if (!ok) break;
                tc_commit(v_empty + 8 * (i & 1));
                if (i + 1 < n_blocks) tc_commit(k_empty + 8 * ((i + 1) & 1));
            }
            if (ok) tc_commit(o_done);
            if (p.trace != nullptr) {
                unsigned long long* at = p.trace + (size_t)blockIdx.x * 16 + 8;
                for (int k = 0; k < 5; ++k) at[k] = m_spent[k];
            }
        }
    } else {
        const int x = (warp - 2) >> 2;                     // this warp's tile
        const int quarter = warp & 3;                      // TMEM lanes this warp may read: 32*quarter ..
        const int r = quarter * 32 + lane;                 // this thread's row of the tile
        const int t = r / G, g = r - t * G;
        const bool valid = active[x] && r < T * G && t0[x] + t < q_len;
        const int pos_r = valid ? pos0 + t0[x] + t : -1;   // -1: every key is masked
        const int lo_r = (valid && p.window > 0) ? max(0, pos_r - p.window + 1) : 0;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const uint32_t tmem_s = tmem_base + 256 * x + lane_addr, tmem_o = tmem_s + 128;
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        int count = 0;                                     // blocks of this tile so far
        unsigned long long spent[5] = {0, 0, 0, 0, 0};
        const bool tracing = p.trace != nullptr && r == 0 && x == 0;
        unsigned long long t_mark = tracing ? global_ns() : 0, t_begin = t_mark;
        auto lap = [&](int which) {
            if (tracing) {
                const unsigned long long now = global_ns();
                spent[which] += now - t_mark;
                t_mark = now;
            }
        };
        for (int i = 0; i < n_blocks && ok && active[x]; ++i) {
            if (!part(x, i)) continue;
            const int b = i & 1, par = (i >> 1) & 1;
            const int kb = ub0 + i;
            const int j0 = kb * KEYS2;
            if (!(ok = mbar_wait(s_full + 8 * x, count & 1, p.status, 6))) break;
            tc_fence_after();
            lap(0);
            const bool need_mask = __any_sync(0xffffffffu, j0 + KEYS2 - 1 > pos0 + t0[x] ||
                                                               (p.window > 0 && j0 < pos_hi[x] - p.window + 1));
            // The row's 128 scores are read from tensor memory once (a load and its wait cost some 400 cycles, whatever
            // the number of columns) and stay in registers for both passes.
            const int hi = pos_r - j0, lo = lo_r - j0;     // columns hi < j or j < lo are masked
            uint32_t raw[KEYS2];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t (&part32)[32] = *reinterpret_cast<uint32_t (*)[32]>(&raw[32 * c]);
                tc_ld32(tmem_s + 32 * c, part32);
            }
            tc_ld_wait();
            if (need_mask) {
#pragma unroll
                for (int j = 0; j < KEYS2; ++j)
                    if (j > hi || j < lo) raw[j] = 0xff800000u;          // -inf
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < KEYS2; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(raw[j]));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
            lap(1);
            // The reference maximum moves only when the true one has grown by more than 8; O is rescaled then.  The
            // tile's second product of the block before is done: this block's scores were issued behind it.
            const bool grow = mx > m_run + 8.f;
            if (__any_sync(0xffffffffu, grow)) {
                const float alpha = grow ? exp2f(m_run - mx) : 1.f;
                if (grow) {
                    m_run = mx;
                    l_run *= alpha;
                }
                if (count > 0) {
#pragma unroll 1
                    for (int c = 0; c < 8; ++c) {
                        if (c * 16 < p.hd) {
                            uint32_t o16[16];
                            tc_ld16(tmem_o + c * 16, o16);
                            tc_ld_wait();
#pragma unroll
                            for (int j = 0; j < 16; ++j) o16[j] = __float_as_uint(__uint_as_float(o16[j]) * alpha);
                            tc_st16(tmem_o + c * 16, o16);
                        }
                    }
                    tc_st_wait();
                }
            }
            lap(3);
            const float neg_m = m_run == -INFINITY ? 0.f : -m_run;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            // P (bf16, two to a column) goes over the first 64 columns of S.
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t packed[32];
#pragma unroll
                for (int j = 0; j < 64; j += 2) {
                    const float e0 = exp2_fast(fmaf(__uint_as_float(raw[64 * h + j]), p.scale_log2, neg_m));
                    const float e1 = exp2_fast(fmaf(__uint_as_float(raw[64 * h + j + 1]), p.scale_log2, neg_m));
                    sum4[j & 2] += e0;
                    sum4[(j & 2) + 1] += e1;
                    packed[j >> 1] = pack2(e0, e1);
                }
                tc_st32(tmem_s + 32 * h, packed);
            }
            tc_st_wait();
            l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            if (kb == ub1) {
                // keys past the last one that any row of the CTA may see: their V rows may hold anything; zero them
                // (both tiles do, each before it hands over its P of this block)
                const int key = j0 + r;
                if (key > pos_hi_u) {
                    if (!(ok = mbar_wait(v_full + 8 * b, par, p.status, 7))) break;
                    for (int s = 0; s < slices; ++s) {
                        uint4* line = (uint4*)(s_v + b * KV_STAGE2 + s * KSLICE2 + r * 128);
#pragma unroll
                        for (int q = 0; q < 8; ++q) line[q] = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            tc_fence_before();
            mbar_arrive(p_full + 8 * x);
            ++count;
            lap(2);
        }
        if (active[x]) {
            if (ok) ok = mbar_wait(o_done, 0, p.status, 8);
            tc_fence_after();
            lap(4);
            if (ok) {
                const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
                bf16* dst = p.out + ((size_t)(q_start + t0[x] + t) * p.nq + (size_t)kvh * G + g) * p.hd;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    if (c * 32 < p.hd) {                               // uniform: the load is warp-wide
                        uint32_t o32[32];
                        tc_ld32(tmem_o + c * 32, o32);
                        tc_ld_wait();
                        if (valid) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                if (c * 32 + q * 8 < p.hd) {
                                    float v[8];
#pragma unroll
                                    for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(o32[q * 8 + j]) * inv;
                                    *(uint4*)(dst + c * 32 + q * 8) =
                                        make_uint4(pack2(v[0], v[1]), pack2(v[2], v[3]), pack2(v[4], v[5]), pack2(v[6], v[7]));
                                }
                            }
                        }
                    }
                }
            }
            if (tracing) {
                unsigned long long* at = p.trace + (size_t)blockIdx.x * 16;
                for (int k = 0; k < 5; ++k) at[k] = spent[k];
                at[5] = (unsigned long long)count;
                at[6] = global_ns() - t_begin;
                at[7] = t_begin;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
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

int encode(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
           const cuuint32_t* box, const char* what) {
    EncodeTiled enc = encode_fn();
    if (enc == nullptr) FR_REFUSE("attention_tc: the driver does not offer cuTensorMapEncodeTiled");
    cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box,
                           estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) FR_REFUSE("attention_tc: cuTensorMapEncodeTiled failed with %d for %s", (int)r, what);
    return FR_OK;
}

constexpr int SMEM_BYTES = 6 * SLICE + 1024 + 256;      // Q, K, V: two 64-dim slices each; two CTAs share an SM

// FRIDAY_ATTN_PAIR=0: prompts always run the kernel with one row tile per CTA.
bool use_pairs() {
    const char* e = getenv("FRIDAY_ATTN_PAIR");
    return e == nullptr || e[0] != '0';
}

}  // namespace

// For measurements: launches after this call record per CTA where the thread of its first row spent its time.
static unsigned long long* attention_tc_trace = nullptr;
FR_EXPORT int attention_tc_set_trace(unsigned long long* trace) {
    attention_tc_trace = trace;
    return FR_OK;
}

// What the kernel takes: bf16, head sizes in steps of 16 up to 128, 64-token pages, at most 128 heads per kv head,
// query rows that start on 16-byte boundaries.
FR_EXPORT int attention_tc_supports(int hd, int page, int nq, int nkv, int q_stride) {
    return hd % 16 == 0 && hd >= 16 && hd <= 128 && page == PAGE && nkv > 0 && nq % nkv == 0 && nq / nkv <= ROWS &&
           q_stride % 8 == 0;
}

// q: rows of q_stride bf16 (head h at h * hd), total_rows of them; out [rows][nq * hd]; pools [pool_pages][64][nkv][hd]
// bf16.  seq_start / seq_qlen / seq_pos0: per sequence, its first row, its rows in this step, the position of its
// first row; seq_live (may be null): indexed by a sequence's first row, negative marks an ended sequence, whose rows
// are left alone.  max_q_len: the longest seq_qlen (sizes the grid).  status: a device word for a wait that gave up.
FR_EXPORT int attention_tc(const void* q, int q_stride, int total_rows, void* out, const void* k_pool, const void* v_pool,
                           int pool_pages, const int* block_table, int table_width, const int* seq_start,
                           const int* seq_qlen, const int* seq_pos0, const int* seq_live, int n_seqs, int max_q_len,
                           int nq, int nkv, int hd, int window, float scale, int* status, cudaStream_t stream) {
    if (n_seqs <= 0 || total_rows <= 0 || max_q_len <= 0) return FR_OK;
    if (!attention_tc_supports(hd, PAGE, nq, nkv, q_stride))
        FR_REFUSE("attention_tc: head size %d, %d heads on %d kv heads, row stride %d: not for this kernel", hd, nq, nkv, q_stride);
    if (((uintptr_t)q & 15) || ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15) || ((uintptr_t)out & 15))
        FR_REFUSE("attention_tc: buffers must be 16-byte aligned");
    if (status == nullptr) FR_REFUSE("attention_tc: a status word is needed");
    const int G = nq / nkv, T = ROWS / G;
    CUtensorMap mq, mk, mv;
    {
        const cuuint64_t dims[4] = {(cuuint64_t)hd, (cuuint64_t)G, (cuuint64_t)nkv, (cuuint64_t)total_rows};
        const cuuint64_t strides[3] = {(cuuint64_t)hd * 2, (cuuint64_t)G * hd * 2, (cuuint64_t)q_stride * 2};
        const cuuint32_t box[4] = {64, (cuuint32_t)G, 1, (cuuint32_t)T};
        const int rc = encode(&mq, q, 4, dims, strides, box, "the queries");
        if (rc) return rc;
    }
    {
        const cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)nkv, (cuuint64_t)pool_pages * PAGE};
        const cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)nkv * hd * 2};
        const cuuint32_t box[3] = {64, 1, PAGE};
        int rc = encode(&mk, k_pool, 3, dims, strides, box, "the keys");
        if (rc) return rc;
        rc = encode(&mv, v_pool, 3, dims, strides, box, "the values");
        if (rc) return rc;
    }
    TcArgs p;
    p.out = (bf16*)out; p.block_table = block_table; p.seq_start = seq_start; p.seq_qlen = seq_qlen;
    p.seq_pos0 = seq_pos0; p.seq_live = seq_live; p.status = status; p.table_width = table_width; p.nq = nq;
    p.nkv = nkv; p.hd = hd; p.window = window; p.pool_rows = pool_pages * PAGE; p.scale_log2 = scale * LOG2E;
    p.trace = attention_tc_trace;
    static bool configured = false;
    if (!configured) {
        FR_CUDA(cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured = true;
    }
    const long long tiles_seq = (max_q_len + T - 1) / T;
    const long long tiles = tiles_seq * nkv * n_seqs;
    if (tiles > 0x7fffffffLL) FR_REFUSE("attention_tc: %lld tiles exceed the grid", tiles);
    p.n_seqs = n_seqs;
    if (tiles_seq >= 2 && use_pairs()) {
        static bool configured2 = false;
        if (!configured2) {
            FR_CUDA(cudaFuncSetAttribute(attention_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES2));
            configured2 = true;
        }
        const dim3 grid((unsigned)(((tiles_seq + 1) / 2) * nkv * n_seqs));
        FR_CUDA(fr_launch(attention_tc_pair_kernel, grid, dim3(THREADS2), SMEM_BYTES2, stream, mq, mk, mv, p));
        FR_CHECK_LAUNCH("attention_tc (two tiles per CTA)");
        return FR_OK;
    }
    const dim3 grid((unsigned)tiles);
    FR_CUDA(fr_launch(attention_tc_kernel, grid, dim3(THREADS), SMEM_BYTES, stream, mq, mk, mv, p));
    FR_CHECK_LAUNCH("attention_tc");
    return FR_OK;
}
