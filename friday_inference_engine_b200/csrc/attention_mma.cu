// Causal grouped-query attention over the paged cache on tensor cores (bf16 operands,
// fp32 scores, softmax and sums), for prompts and for decoding.
//
// The query heads that share one key/value head are packed into the rows of one tile:
// for a sequence and a kv head, row r stands for (token r / G, group head r % G), G =
// heads / kv heads.  A key/value block is then read once for all G heads, which is what
// makes decoding with grouped heads memory-bound instead of compute-bound (the reference
// does the same with CUDA cores: decodeAttentionGqaKernel, attention_kernels.cu:267-411,
// and its R = tq*G + g rows for prompts, :493-499).
//
// Blocks of 64 keys are exactly the cache's pages, so a block is one page lookup.  Fragments come from ldmatrix,
// products are mma.sync.m16n8k16 with the online softmax of flash attention between them.  How K and V blocks
// get from global to shared memory differs:
//   prompts          cp.async by the computing warps into padded rows, two buffers; rows past a sequence's last
//                    needed key are zero-filled;
//   one-token steps  a fifth warp issues TMA loads of whole pages (64 keys x 64 dims a box, 128-byte swizzle) into a
//                    ring of three blocks with an mbarrier per buffer; ldmatrix addresses undo the swizzle; the
//                    computing warps issue no copies and meet no block-wide barrier in the loop.  Blocks of earlier
//                    steps are requested before the wait for the kernel before this one.  V rows past the last
//                    needed key are zeroed in shared memory (a zero weight times a stale NaN is a NaN); scores of
//                    such keys are replaced by the mask.
//
// Two shapes of the same kernel:
//   rows mode (prompts): a CTA owns 64 rows; each of its 4 warps owns 16 rows and walks
//       all 64 keys of a block;
//   keys mode (decoding): a CTA owns 16 rows (one token's G heads, padded) and a range of
//       blocks (`splits` CTAs share a sequence's keys); each warp takes 16 of a block's 64
//       keys; warps merge through shared memory; the splits of a tile form a thread-block
//       cluster and merge through each other's shared memory (more than 8 splits: through
//       a scratch buffer, the last CTA to arrive merging).
// Head sizes: multiples of 16 up to 128.  Others are served by the CUDA-core kernel.
#include <math.h>

#include "attention_merge.cuh"
#include "common.cuh"
#include "tc_common.cuh"

FR_EXPORT const char* attention_mma_last_error() { return fr_error_text; }

namespace {

typedef __nv_bfloat16 bf16;
constexpr int BLOCK_N = 64;     // keys per block = tokens per cache page
constexpr int WARPS = 4;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

struct MmaArgs {
    const bf16* q;            // rows of q_stride elements; head h at h * hd
    bf16* out;                // [rows][nq * hd]
    const bf16* k_pool;       // [pages][64][nkv][hd]
    const bf16* v_pool;
    const int* block_table;   // [seqs][table_width]
    const int* seq_start;     // first row of each sequence
    const int* seq_qlen;      // rows (tokens) of each sequence in this step
    const int* seq_pos0;      // position of its first row
    const int* seq_live;      // may be null; < 0 at seq_start[s]: the sequence has ended (row marker)
    float* part;              // [rows * nq][splits][hd + 2] when splits > 1
    int* counters;            // keys mode with splits: one per (sequence, kv head, row tile), zero between launches;
                              // the CTA that finishes a tile's last split merges the splits itself
    int cluster;              // keys mode: the `splits` CTAs of a tile form a thread-block cluster and merge through
                              // each other's shared memory (no scratch, no counters)
    int q_stride, table_width, nq, nkv, window, splits;
    float scale_log2;         // softmax scale times log2(e)
    int pool_rows;            // rows of a pool (pages x 64): a load from there on is filled with zeros
    int* status;              // a word that receives a code when a bounded wait of the one-token kernel gave up
    unsigned long long* trace;  // for measurements (may be null): [cta][8] timestamps of a one-token step's CTAs
};

__device__ __forceinline__ void mark(const MmaArgs& p, int point) {
    if (p.trace != nullptr && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        p.trace[((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8 + point] = t;
    }
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

// One-token steps have a fifth warp that only copies: it keeps the ring of K/V blocks full with TMA loads of whole
// pages (one instruction per 64 keys x 64 dims, 128-byte swizzle, completion on an mbarrier), so the four computing
// warps issue no copy instructions and meet no block-wide barrier inside the loop.  (Bulk copies of single rows, one
// instruction per 256 bytes, were three times slower than the cp.async of the computing warps.)
__device__ __forceinline__ void tma_page(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}

template <int HD, bool KEYS_MODE>
__global__ void __launch_bounds__(KEYS_MODE ? (WARPS + 1) * 32 : WARPS * 32)
attention_mma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const MmaArgs p) {
    constexpr int ROW_BYTES = HD * 2 + 16;            // padded: 8 consecutive rows hit 8 different bank groups
    constexpr int CHUNKS = HD / 8;                    // 16-byte pieces per row
    constexpr int ROWS_CTA = KEYS_MODE ? 16 : 64;
    constexpr int KPW = KEYS_MODE ? 16 : 64;          // keys of a block per warp
    constexpr int NT = KPW / 8;                       // score tiles (8 keys each) per warp
    constexpr int DT = HD / 8;                        // output tiles (8 dims each)
    // Buffers of the K/V ring.  One-token steps do almost no arithmetic per block, so what bounds them is how many
    // blocks are on their way from memory: three buffers keep two in flight; prompts are bound by arithmetic.
    constexpr int NS = KEYS_MODE ? 3 : 2;
    // One-token steps: a block's keys (and values) lie as SL slices of 64 dims, each [64 keys][128 bytes] with the
    // 16-byte pieces of a row exchanged by the row's number (TMA's 128-byte swizzle), behind a 1 KB boundary.
    constexpr int SL = (HD + 63) / 64;
    constexpr int KV_BYTES = KEYS_MODE ? SL * BLOCK_N * 128 : BLOCK_N * ROW_BYTES;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint8_t* smem = KEYS_MODE ? (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023) : smem_raw;
    uint8_t* s_k = smem;                              // [NS] blocks
    uint8_t* s_v = s_k + NS * KV_BYTES;               // [NS] blocks
    uint8_t* s_q = s_v + NS * KV_BYTES;               // [ROWS_CTA][ROW_BYTES]

    __shared__ int s_pages[WARPS * 32];               // the sequence's first pages, read before anything depends on them
    __shared__ uint64_t s_bars[2 * NS];               // one-token steps: full[NS], empty[NS]
    const uint32_t full0 = tc::smem_u32(s_bars), empty0 = tc::smem_u32(s_bars + NS);
    if (KEYS_MODE && threadIdx.x == 0) {
        for (int b = 0; b < NS; ++b) {
            tc::mbar_init(full0 + 8 * b, 1);
            tc::mbar_init(empty0 + 8 * b, WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    mark(p, 0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = blockIdx.z, kvh = blockIdx.y;
    // The page table is written by copies from the host, never by a kernel, so it may be read before the
    // kernel before this one has finished; so may everything that is arithmetic only.  The rest waits.
    // (s_pages holds the first WARPS * 32 entries; keys mode runs one warp more than that, whose threads must not store)
    if (tid < p.table_width && tid < WARPS * 32) s_pages[tid] = p.block_table[(size_t)seq * p.table_width + tid];
    const int split = blockIdx.x % p.splits, tile = blockIdx.x / p.splits;
    const int G = p.nq / p.nkv;
    const int r0 = tile * ROWS_CTA;
    const int* table = p.block_table + (size_t)seq * p.table_width;
    const size_t kv_row = (size_t)p.nkv * HD;         // elements between consecutive keys of a page
    // Which pieces of a K/V block this thread copies is the same for every block: row, source offset and
    // destination offset are worked out once.
    constexpr int PIECES = BLOCK_N * CHUNKS / (WARPS * 32);
    int piece_row[PIECES], piece_src[PIECES], piece_dst[PIECES];
#pragma unroll
    for (int j = 0; j < PIECES; ++j) {
        const int c = tid + j * WARPS * 32;
        const int r = c / CHUNKS, ch = c - r * CHUNKS;
        piece_row[j] = r;
        piece_src[j] = r * (int)kv_row + ch * 8;
        piece_dst[j] = r * ROW_BYTES + ch * 16;
    }
    const uint32_t k_smem = (uint32_t)__cvta_generic_to_shared(s_k), v_smem = (uint32_t)__cvta_generic_to_shared(s_v);
    // The step's geometry (rows, positions, which sequences have ended) is written before the step's first kernel
    // starts, by copies from the host or by the step before, and every step begins with kernels that wait for
    // their predecessor before they let a dependent launch (common.cuh): it, too, is read ahead of the wait.
    const int q_len = p.seq_qlen[seq], q_start = p.seq_start[seq], pos0 = p.seq_pos0[seq];
    const int n_rows = q_len * G;
    const bool live = p.seq_live == nullptr || p.seq_live[q_start] >= 0;
    __syncthreads();                                   // s_pages

    // Range of key blocks for this CTA.
    const int t_first = r0 / G, t_last = min((r0 + ROWS_CTA - 1) / G, q_len - 1);
    const int pos_hi = pos0 + t_last;                 // the farthest key any row of the CTA may see
    const int lo_min = p.window > 0 ? max(0, pos0 + t_first - p.window + 1) : 0;
    int kb_begin = lo_min / BLOCK_N, kb_end = pos_hi / BLOCK_N;     // inclusive
    if (p.splits > 1) {
        const int n = kb_end - kb_begin + 1, per = (n + p.splits - 1) / p.splits;
        kb_begin += split * per;
        kb_end = min(kb_begin + per - 1, kb_end);
    }
    if (!live || r0 >= n_rows) kb_end = kb_begin - 1;  // nothing to read: the output is zero (or there is none)

    auto load_q = [&]() {
        for (int c = tid; c < ROWS_CTA * CHUNKS; c += WARPS * 32) {
            const int r = c / CHUNKS, ch = c - r * CHUNKS;
            const int rr = r0 + r;
            const bool ok = rr < n_rows;
            const int t = ok ? rr / G : 0, g = ok ? rr - t * G : 0;
            const bf16* src = p.q + (size_t)(q_start + t) * p.q_stride + (size_t)(kvh * G + g) * HD + ch * 8;
            cp_async16((uint32_t)__cvta_generic_to_shared(s_q + r * ROW_BYTES + ch * 16), src, ok ? 16 : 0);
        }
    };
    auto load_kv = [&](int kb, int buf) {
        const int page = kb < WARPS * 32 ? s_pages[kb] : table[kb];
        const bf16* kbase = p.k_pool + ((size_t)page * BLOCK_N) * kv_row + (size_t)kvh * HD;
        const bf16* vbase = p.v_pool + ((size_t)page * BLOCK_N) * kv_row + (size_t)kvh * HD;
        // rows of the block that are needed; none of a page that the table does not name (a sequence that has ended)
        const int valid = page >= 0 ? pos_hi - kb * BLOCK_N + 1 : 0;
#pragma unroll
        for (int j = 0; j < PIECES; ++j) {
            const bool ok = piece_row[j] < valid;                           // beyond the last needed key: zeros
            cp_async16(k_smem + buf * KV_BYTES + piece_dst[j], ok ? (const void*)(kbase + piece_src[j]) : (const void*)p.k_pool,
                       ok ? 16 : 0);
            cp_async16(v_smem + buf * KV_BYTES + piece_dst[j], ok ? (const void*)(vbase + piece_src[j]) : (const void*)p.v_pool,
                       ok ? 16 : 0);
        }
    };

    // Keys and values of earlier steps are final before this step's first kernel starts; only the blocks from the
    // step's own first position on are written by the kernel before this one.  The copying warp of a one-token step
    // therefore starts at once and waits for the kernel before only when it reaches such a block.
    const int first_fresh = pos0 / BLOCK_N;            // blocks from here on hold rows of this step
    const bool producer = KEYS_MODE && warp == WARPS;
    if (producer) {
        bool waited = false, ok = true;
        int j = 0;
        for (int kb = kb_begin; kb <= kb_end && ok; ++kb, ++j) {
            const int b = j % NS;
            if (kb >= first_fresh && !waited) {
                fr_pdl_wait();
                waited = true;
            }
            if (!(ok = tc::mbar_wait(empty0 + 8 * b, ((j / NS) & 1) ^ 1, p.status, 21))) break;
            const int page = kb < WARPS * 32 ? s_pages[kb] : table[kb];
            if (tc::elect_one()) {
                // a page that the table does not name is loaded from beyond the pool's last row: zeros
                const int row = page >= 0 ? page * BLOCK_N : p.pool_rows;
                tc::mbar_expect_tx(full0 + 8 * b, (uint32_t)(2 * SL * BLOCK_N * 128));
                for (int sl = 0; sl < SL; ++sl) {
                    tma_page(k_smem + b * KV_BYTES + sl * BLOCK_N * 128, &map_k, sl * 64, kvh, row, full0 + 8 * b);
                    tma_page(v_smem + b * KV_BYTES + sl * BLOCK_N * 128, &map_v, sl * 64, kvh, row, full0 + 8 * b);
                }
            }
            __syncwarp();
        }
        if (!waited) fr_pdl_wait();
        fr_pdl_launch();
    } else {
        fr_pdl_wait();
        fr_pdl_launch();
    }
    mark(p, 1);
    if (r0 >= n_rows) return;

    // This thread's two rows (fragment layout of mma: rows lane/4 and lane/4 + 8 of the warp's 16).
    const int row_base = KEYS_MODE ? 0 : warp * 16;
    const int key_base = KEYS_MODE ? warp * 16 : 0;
    int pos_r[2], lo_r[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int rr = r0 + row_base + (lane >> 2) + 8 * i;
        const bool ok = rr < n_rows;
        pos_r[i] = ok ? pos0 + rr / G : -1;           // -1: every key is masked
        lo_r[i] = (ok && p.window > 0) ? max(0, pos_r[i] - p.window + 1) : 0;
    }
    // Warp-wide bounds that decide whether a block needs the mask at all.
    const int w_first = (r0 + row_base) / G;
    const int w_last = min((r0 + row_base + 15) / G, q_len - 1);
    const int w_pos_min = pos0 + w_first;
    const int w_lo_max = p.window > 0 ? max(0, pos0 + w_last - p.window + 1) : 0;

    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; ++d)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[d][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    if (!producer) load_q();
    if (!KEYS_MODE) {
#pragma unroll
        for (int st = 0; st < NS - 1; ++st)
            if (kb_begin + st <= kb_end) load_kv(kb_begin + st, st);
    }
    cp_commit();                                       // the queries (and for prompts the first blocks)
    if (KEYS_MODE) {
        cp_wait<0>();
        if (!producer) asm volatile("bar.sync 1, %0;" ::"n"(WARPS * 32) : "memory");     // the queries are in place
    }

    mark(p, 2);
    const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(s_q);
    uint32_t q_frag[KEYS_MODE ? HD / 16 : 1][4];       // one-token steps keep the queries in registers
    bool q_loaded = false;
    int buf = 0;
    bool ring_ok = true;
    int round = 0;                                     // how often the ring has gone round
    for (int kb = producer ? kb_end + 1 : kb_begin; kb <= kb_end && ring_ok; ++kb) {
        if (KEYS_MODE) {
            if (!(ring_ok = tc::mbar_wait(full0 + 8 * buf, round & 1, p.status, 22))) break;
            const int valid = pos_hi - kb * BLOCK_N + 1;
            if (kb == kb_end && valid < BLOCK_N) {
                // rows past the last needed key come with the page: what lies there may be anything, and a zero weight
                // times a NaN is a NaN.  Zero those rows of V (scores of such keys are replaced by the mask).
                for (int c = tid; c < (BLOCK_N - valid) * SL * 8; c += WARPS * 32) {
                    const int r = valid + c / (SL * 8), rest = c % (SL * 8);
                    *(uint4*)(s_v + buf * KV_BYTES + (rest >> 3) * BLOCK_N * 128 + r * 128 + (rest & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
                }
                asm volatile("bar.sync 1, %0;" ::"n"(WARPS * 32) : "memory");
            }
        } else {
            const int ahead = buf + NS - 1 >= NS ? buf - 1 : buf + NS - 1;      // the buffer used one block ago
            if (kb + NS - 1 <= kb_end) load_kv(kb + NS - 1, ahead);
            cp_commit();
            cp_wait<NS - 1>();                         // everything but the newest NS-1 groups: block kb is here
            __syncthreads();
        }
        if (kb == kb_begin) mark(p, 3);
        const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(s_k + buf * KV_BYTES);
        const uint32_t v_addr = (uint32_t)__cvta_generic_to_shared(s_v + buf * KV_BYTES);

        // scores = Q K^T for this warp's 16 rows and KPW keys
        float s[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
        if (KEYS_MODE && !q_loaded) {
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks)
                ldsm4(q_frag[ks], q_addr + (row_base + (lane & 7) + 8 * ((lane >> 3) & 1)) * ROW_BYTES +
                                      (ks * 16 + 8 * (lane >> 4)) * 2);
            q_loaded = true;
        }
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            uint32_t a_now[4];
            if (!KEYS_MODE)
                ldsm4(a_now, q_addr + (row_base + (lane & 7) + 8 * ((lane >> 3) & 1)) * ROW_BYTES + (ks * 16 + 8 * (lane >> 4)) * 2);
            const uint32_t (&a)[4] = KEYS_MODE ? q_frag[ks] : a_now;
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                uint32_t b[4];
                const int krow = key_base + np * 16 + (lane & 7) + 8 * (lane >> 4), kch = ks * 2 + ((lane >> 3) & 1);
                ldsm4(b, KEYS_MODE ? k_addr + (kch >> 3) * BLOCK_N * 128 + krow * 128 + (((kch & 7) ^ (krow & 7)) << 4)
                                   : k_addr + krow * ROW_BYTES + kch * 16);
                mma16816(s[2 * np], a, b[0], b[1]);
                mma16816(s[2 * np + 1], a, b[2], b[3]);
            }
        }

        // scale, mask, online softmax
        const int j0 = kb * BLOCK_N + key_base;
        const bool need_mask = (j0 + KPW - 1 > w_pos_min) || (p.window > 0 && j0 < w_lo_max);
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[n][e] * p.scale_log2;
                if (need_mask) {
                    const int j = j0 + n * 8 + 2 * (lane & 3) + (e & 1);
                    if (j > pos_r[e >> 1] || j < lo_r[e >> 1]) v = -INFINITY;
                } else if (pos_r[e >> 1] < 0) {
                    v = -INFINITY;
                }
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
            alpha[i] = exp2f(m_run[i] - m_use[i]);     // 0 while the row has seen no key
            m_run[i] = m_new;
        }
        float sum[2] = {0.f, 0.f};
#pragma unroll
        for (int n = 0; n < NT; ++n)
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

        // o += P V
#pragma unroll
        for (int kk = 0; kk < KPW / 16; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < DT / 2; ++dp) {
                uint32_t b[4];
                const int vrow = key_base + kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), vch = dp * 2 + (lane >> 4);
                ldsm4_t(b, KEYS_MODE ? v_addr + (vch >> 3) * BLOCK_N * 128 + vrow * 128 + (((vch & 7) ^ (vrow & 7)) << 4)
                                     : v_addr + vrow * ROW_BYTES + vch * 16);
                mma16816(o[2 * dp], a, b[0], b[1]);
                mma16816(o[2 * dp + 1], a, b[2], b[3]);
            }
        }
        if (KEYS_MODE) {
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(empty0 + 8 * buf);      // this warp is done with the buffer
        } else {
            __syncthreads();      // every warp is done with this buffer before it is loaded again
        }
        if (++buf == NS) {
            buf = 0;
            ++round;
        }
    }
    cp_wait<0>();
    mark(p, 4);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }

    if (!KEYS_MODE) {
        // Each warp owns its rows outright.
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int rr = r0 + row_base + (lane >> 2) + 8 * i;
            if (rr >= n_rows) continue;
            const int t = rr / G, h = kvh * G + (rr - t * G);
            const size_t item = (size_t)(q_start + t) * p.nq + h;
            if (p.splits == 1) {
                const float inv = l_run[i] > 0.f ? 1.f / l_run[i] : 0.f;
                bf16* dst = p.out + item * HD;
#pragma unroll
                for (int d = 0; d < DT; ++d)
                    *reinterpret_cast<uint32_t*>(dst + d * 8 + 2 * (lane & 3)) =
                        pack_bf16(o[d][2 * i] * inv, o[d][2 * i + 1] * inv);
            } else {
                float* dst = p.part + (item * p.splits + split) * (HD + 2);
#pragma unroll
                for (int d = 0; d < DT; ++d) {
                    dst[d * 8 + 2 * (lane & 3)] = o[d][2 * i];
                    dst[d * 8 + 2 * (lane & 3) + 1] = o[d][2 * i + 1];
                }
                if ((lane & 3) == 0) {
                    dst[HD] = m_run[i] * LN2;
                    dst[HD + 1] = l_run[i];
                }
            }
        }
    } else {
        // The four warps saw different keys of the same 16 rows: merge through shared memory
        // (the K/V buffers are free now).
        constexpr int HDP = HD + 4;                                 // padded: the 8 rows of a warp's store hit 8 bank groups
        float* c_o = reinterpret_cast<float*>(s_k);                 // [WARPS][16][HDP]
        float* c_m = c_o + WARPS * 16 * HDP;                        // [WARPS][16]
        float* c_l = c_m + WARPS * 16;
        float* r_o = c_l + WARPS * 16;                              // [16][HD]: this CTA's merged rows (cluster path)
        float* r_m = r_o + 16 * HD;                                 // [16]
        float* r_l = r_m + 16;
        __syncthreads();                              // every warp is done with the last K/V buffers
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = (lane >> 2) + 8 * i;
            if (producer) break;
#pragma unroll
            for (int d = 0; d < DT; ++d) {
                *reinterpret_cast<float2*>(c_o + (warp * 16 + r) * HDP + d * 8 + 2 * (lane & 3)) = make_float2(o[d][2 * i], o[d][2 * i + 1]);
            }
            if ((lane & 3) == 0) {
                c_m[warp * 16 + r] = m_run[i];
                c_l[warp * 16 + r] = l_run[i];
            }
        }
        __syncthreads();
        const int r = tid >> 3;                       // 16 rows x 8 threads (the copying warp has none)
        const int rr = producer ? n_rows : r0 + r;
        if (rr < n_rows) {
            float big = -INFINITY;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) big = fmaxf(big, c_m[w * 16 + r]);
            float f[WARPS], l = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                f[w] = c_m[w * 16 + r] == -INFINITY ? 0.f : exp2f(c_m[w * 16 + r] - big);
                l += c_l[w * 16 + r] * f[w];
            }
            const int t = rr / G, h = kvh * G + (rr - t * G);
            const size_t item = (size_t)(q_start + t) * p.nq + h;
            const float inv = l > 0.f ? 1.f / l : 0.f;
            // A row's eight threads take HD / 8 consecutive dimensions each, in pieces of four (two for head sizes
            // that are no multiple of 32): all loads of a piece's four warps are issued before the first is used (one
            // dimension at a time, this loop took 1.6 us of a 9 us kernel).
            constexpr int PER = HD / 8;                  // 2, 4, ... 16
            constexpr int V = PER % 4 == 0 ? 4 : 2;      // floats per piece
            const int d0 = (tid & 7) * PER;
#pragma unroll
            for (int c = 0; c < PER / V; ++c) {
                float acc[V];
#pragma unroll
                for (int j = 0; j < V; ++j) acc[j] = 0.f;
#pragma unroll
                for (int w = 0; w < WARPS; ++w) {
                    const float* src = c_o + (w * 16 + r) * HDP + d0 + c * V;
                    if (V == 4) {
                        const float4 x = *reinterpret_cast<const float4*>(src);
                        acc[0] += x.x * f[w]; acc[1] += x.y * f[w]; acc[2 % V] += x.z * f[w]; acc[3 % V] += x.w * f[w];
                    } else {
                        const float2 x = *reinterpret_cast<const float2*>(src);
                        acc[0] += x.x * f[w]; acc[1] += x.y * f[w];
                    }
                }
                const int d = d0 + c * V;
                if (p.splits == 1) {
#pragma unroll
                    for (int j = 0; j < V; j += 2)
                        *reinterpret_cast<uint32_t*>(p.out + item * HD + d + j) = pack_bf16(acc[j] * inv, acc[j + 1] * inv);
                } else {
                    float* dst = p.cluster ? r_o + r * HD + d : p.part + (item * p.splits + split) * (HD + 2) + d;
#pragma unroll
                    for (int j = 0; j < V; j += 2) *reinterpret_cast<float2*>(dst + j) = make_float2(acc[j], acc[j + 1]);
                }
            }
            if (p.cluster && p.splits > 1 && (tid & 7) == 0) {
                r_m[r] = big;
                r_l[r] = l;
            }
            if (!p.cluster && p.splits > 1 && (tid & 7) == 0) {
                float* dst = p.part + (item * p.splits + split) * (HD + 2);
                dst[HD] = big * LN2;                  // natural-log units, as the merge kernel expects
                dst[HD + 1] = l;
            }
        }
        if (p.splits > 1 && p.cluster) {
            // The splits of this tile are the CTAs of one cluster.  Every CTA merges a share of the 16 rows, reading
            // all CTAs' merged rows from their shared memory, four dimensions per thread and pass; all loads of a
            // pass are issued before the first is used, so a pass costs one trip through the cluster's network, not
            // one per load.  Nothing goes through global memory.
            mark(p, 5);
            fr_cluster_sync();
            mark(p, 6);
            const int rank = (int)fr_cluster_rank();
            const int rows_per = (16 + p.splits - 1) / p.splits;
            constexpr int VEC = HD / 4;                                 // float4 pieces per row
            for (int idx = producer ? rows_per * VEC : tid; idx < rows_per * VEC; idx += WARPS * 32) {
                const int r2 = rank * rows_per + idx / VEC, d4 = idx % VEC;
                const int rr2 = r0 + r2;
                if (r2 >= 16 || rr2 >= n_rows) continue;
                float ms[8], ls[8];
                float4 vs[8];
#pragma unroll
                for (int sp = 0; sp < 8; ++sp) {
                    if (sp < p.splits) {
                        ms[sp] = fr_cluster_load(r_m + r2, sp);
                        ls[sp] = fr_cluster_load(r_l + r2, sp);
                        vs[sp] = fr_cluster_load4(r_o + r2 * HD + d4 * 4, sp);
                    } else {
                        ms[sp] = -INFINITY;
                        ls[sp] = 0.f;
                        vs[sp] = make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
                float big = -INFINITY;
#pragma unroll
                for (int sp = 0; sp < 8; ++sp) big = fmaxf(big, ms[sp]);
                float l = 0.f;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int sp = 0; sp < 8; ++sp) {
                    const float f = ms[sp] == -INFINITY ? 0.f : exp2f(ms[sp] - big);
                    l += ls[sp] * f;
                    acc.x += vs[sp].x * f; acc.y += vs[sp].y * f; acc.z += vs[sp].z * f; acc.w += vs[sp].w * f;
                }
                const int t = rr2 / G, h = kvh * G + (rr2 - t * G);
                const size_t item = (size_t)(q_start + t) * p.nq + h;
                const float inv = l > 0.f ? 1.f / l : 0.f;
                uint2 packed;
                packed.x = pack_bf16(acc.x * inv, acc.y * inv);
                packed.y = pack_bf16(acc.z * inv, acc.w * inv);
                *reinterpret_cast<uint2*>(p.out + item * HD + d4 * 4) = packed;
            }
            mark(p, 7);
            fr_cluster_sync();                        // nobody leaves while another CTA still reads its shared memory
        } else if (p.splits > 1 && p.counters != nullptr) {
            // Whoever writes a tile's last partial merges them: no second kernel, the partials are still in L2.
            __shared__ int s_last;
            mark(p, 5);
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                int* c = p.counters + ((size_t)seq * p.nkv + kvh) * (gridDim.x / p.splits) + tile;
                s_last = atomicAdd(c, 1) == p.splits - 1;
                if (s_last) *c = 0;                   // ready for the next launch
            }
            __syncthreads();
            if (s_last) {
                mark(p, 6);
                __threadfence();
                // All splits' partial rows are in L2.  A trip there takes as long for one load as for dozens, so each
                // phase asks for everything it needs at once: first every split's maximum and sum, then the rows
                // themselves, the splits dealt out over the warps and a row's dimensions over a warp's lanes.
                const int S = p.splits;                             // at most 64 on this path
                const int n_here = min(16, n_rows - r0);
                float* red = c_o;                                   // [WARPS][16][HD]: each warp's share of the sums
                float* s_w = red + WARPS * 16 * HD;                 // [16][64]: a split's maximum, then its weight exp(m - M)
                float* s_ls = s_w + 16 * 64;                        // [16][64]: a split's sum
                float* s_inv = s_ls + 16 * 64;                      // [16]: one over a row's sum
                auto part_of = [&](int r2) -> const float* {
                    const int rr2 = r0 + r2, t2 = rr2 / G, h2 = kvh * G + (rr2 - t2 * G);
                    return p.part + ((size_t)(q_start + t2) * p.nq + h2) * S * (HD + 2);
                };
                for (int idx = tid; idx < n_here * S; idx += blockDim.x) {
                    const int r2 = idx / S, sp = idx - r2 * S;
                    const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_of(r2) + (size_t)sp * (HD + 2) + HD));
                    s_w[r2 * 64 + sp] = ml.x;
                    s_ls[r2 * 64 + sp] = ml.y;
                }
                __syncthreads();
                {
                    const bool valid = r < n_here;                  // 8 threads per row; the copying warp has none
                    float big = -INFINITY;
                    if (valid)
                        for (int sp = tid & 7; sp < S; sp += 8) big = fmaxf(big, s_w[r * 64 + sp]);
#pragma unroll
                    for (int o2 = 1; o2 < 8; o2 <<= 1) big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, o2));
                    float l = 0.f;
                    if (valid)
                        for (int sp = tid & 7; sp < S; sp += 8) {
                            const float ls = s_ls[r * 64 + sp];
                            const float f = ls > 0.f ? expf(s_w[r * 64 + sp] - big) : 0.f;
                            s_w[r * 64 + sp] = f;
                            l += ls * f;
                        }
#pragma unroll
                    for (int o2 = 1; o2 < 8; o2 <<= 1) l += __shfl_xor_sync(0xffffffffu, l, o2);
                    if (valid && (tid & 7) == 0) s_inv[r] = l > 0.f ? 1.f / l : 0.f;
                }
                __syncthreads();
                constexpr int MPIECES = HD / 2;                      // float2 pieces of a row
                constexpr int PP = (MPIECES + 31) / 32;              // pieces per lane
                if (warp < WARPS) {
#pragma unroll 1
                    for (int half = 0; half < 16; half += 8) {
                        float2 acc[8][PP];
#pragma unroll
                        for (int i = 0; i < 8; ++i)
#pragma unroll
                            for (int j = 0; j < PP; ++j) acc[i][j] = make_float2(0.f, 0.f);
                        if (half < n_here) {
                            // Straight-line code, so that all loads of a pass are on their way before the first is
                            // used: rows beyond the tile's last read that row again and count for nothing.
                            const float* bases[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const bool in = half + i < n_here;
                                bases[i] = part_of(in ? half + i : n_here - 1);
                            }
#pragma unroll 2
                            for (int sp = warp; sp < S; sp += WARPS) {
                                float2 v[8][PP];
#pragma unroll
                                for (int i = 0; i < 8; ++i)
#pragma unroll
                                    for (int j = 0; j < PP; ++j) {
                                        const int piece = lane + 32 * j;
                                        v[i][j] = piece < MPIECES
                                                      ? __ldcg(reinterpret_cast<const float2*>(bases[i] + (size_t)sp * (HD + 2)) + piece)
                                                      : make_float2(0.f, 0.f);
                                    }
#pragma unroll
                                for (int i = 0; i < 8; ++i) {
                                    const float f = half + i < n_here ? s_w[(half + i) * 64 + sp] : 0.f;
#pragma unroll
                                    for (int j = 0; j < PP; ++j) {
                                        acc[i][j].x += v[i][j].x * f;
                                        acc[i][j].y += v[i][j].y * f;
                                    }
                                }
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i)
#pragma unroll
                            for (int j = 0; j < PP; ++j) {
                                const int piece = lane + 32 * j;
                                if (piece < MPIECES) *reinterpret_cast<float2*>(red + (warp * 16 + half + i) * HD + 2 * piece) = acc[i][j];
                            }
                    }
                }
                __syncthreads();
                for (int idx = tid; idx < n_here * MPIECES; idx += blockDim.x) {
                    const int r2 = idx / MPIECES, piece = idx - r2 * MPIECES;
                    float2 a = make_float2(0.f, 0.f);
#pragma unroll
                    for (int w = 0; w < WARPS; ++w) {
                        const float2 v = *reinterpret_cast<const float2*>(red + (w * 16 + r2) * HD + 2 * piece);
                        a.x += v.x;
                        a.y += v.y;
                    }
                    const float inv = s_inv[r2];
                    const int rr2 = r0 + r2, t2 = rr2 / G, h2 = kvh * G + (rr2 - t2 * G);
                    *reinterpret_cast<uint32_t*>(p.out + ((size_t)(q_start + t2) * p.nq + h2) * HD + 2 * piece) =
                        pack_bf16(a.x * inv, a.y * inv);
                }
                mark(p, 7);
            }
        }
    }
}

// FRIDAY_ATTN_CLUSTER=0 merges the splits through global memory instead (for comparison).
bool use_clusters() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("FRIDAY_ATTN_CLUSTER");
        v = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

// Dynamic shared memory: the K/V ring (one-token steps: 128-byte rows per 64-dim slice behind a 1 KB boundary;
// prompts: padded rows) or, if larger, what the merge of a one-token step's warps needs; and the queries.
template <int HD, bool KEYS_MODE>
constexpr int smem_bytes() {
    constexpr int ROW_BYTES = HD * 2 + 16;
    constexpr int ROWS_CTA = KEYS_MODE ? 16 : 64;
    constexpr int kv = KEYS_MODE ? 2 * 3 * ((HD + 63) / 64) * BLOCK_N * 128 : 2 * 2 * BLOCK_N * ROW_BYTES;
    constexpr int merge = KEYS_MODE ? (WARPS * 16 * (HD + 4) + 2 * WARPS * 16 + 16 * HD + 32) * 4 : 0;
    return (KEYS_MODE ? 1024 : 0) + ROWS_CTA * ROW_BYTES + (kv > merge ? kv : merge);
}

template <int HD, bool KEYS_MODE>
int launch(const CUtensorMap& mk, const CUtensorMap& mv, const MmaArgs& p, dim3 grid, cudaStream_t stream) {
    constexpr int smem = smem_bytes<HD, KEYS_MODE>();
    static bool configured = false;
    if (!configured) {
        FR_CUDA(cudaFuncSetAttribute(attention_mma_kernel<HD, KEYS_MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured = true;
    }
    FR_CUDA(fr_launch_cluster(attention_mma_kernel<HD, KEYS_MODE>, grid, dim3(KEYS_MODE ? (WARPS + 1) * 32 : WARPS * 32), smem,
                              stream, p.cluster ? (unsigned)p.splits : 1u, mk, mv, p));
    FR_CHECK_LAUNCH("attention_mma");
    return FR_OK;
}

// Clusters of `size` CTAs of the one-token kernel that the device runs at once (0 if the query fails).
template <int HD>
int clusters_at_once(int size) {
    static int known[9] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};
    if (size < 1 || size > 8) return 0;
    if (known[size] < 0) {
        known[size] = 0;
        constexpr int smem = smem_bytes<HD, true>();
        if (cudaFuncSetAttribute(attention_mma_kernel<HD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(size * 64);
            cfg.blockDim = dim3((WARPS + 1) * 32);
            cfg.dynamicSmemBytes = smem;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = size;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, attention_mma_kernel<HD, true>, &cfg) == cudaSuccess) known[size] = n;
        }
        cudaGetLastError();
    }
    return known[size];
}

template <bool KEYS_MODE>
int launch_hd(int hd, const CUtensorMap& mk, const CUtensorMap& mv, const MmaArgs& p, dim3 grid, cudaStream_t stream) {
    switch (hd) {
        case 16: return launch<16, KEYS_MODE>(mk, mv, p, grid, stream);
        case 32: return launch<32, KEYS_MODE>(mk, mv, p, grid, stream);
        case 48: return launch<48, KEYS_MODE>(mk, mv, p, grid, stream);
        case 64: return launch<64, KEYS_MODE>(mk, mv, p, grid, stream);
        case 80: return launch<80, KEYS_MODE>(mk, mv, p, grid, stream);
        case 96: return launch<96, KEYS_MODE>(mk, mv, p, grid, stream);
        case 112: return launch<112, KEYS_MODE>(mk, mv, p, grid, stream);
        case 128: return launch<128, KEYS_MODE>(mk, mv, p, grid, stream);
        default: FR_REFUSE("attention_mma: head size %d is not built (multiples of 16 up to 128)", hd);
    }
}

// A pool [pages][64][nkv][hd] as a 3-d tensor (dims, kv heads, rows); boxes of 64 dims x 64 rows, 128-byte swizzle.
int pool_map(CUtensorMap* map, const void* pool, int pool_pages, int nkv, int hd) {
    typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeTiled enc = nullptr;
    if (enc == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            enc = (EncodeTiled)ptr;
    }
    if (enc == nullptr) FR_REFUSE("attention_mma: the driver does not offer cuTensorMapEncodeTiled");
    const cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)nkv, (cuuint64_t)pool_pages * BLOCK_N};
    const cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)nkv * hd * 2};
    const cuuint32_t box[3] = {64, 1, BLOCK_N};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(pool), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) FR_REFUSE("attention_mma: cuTensorMapEncodeTiled failed with %d", (int)r);
    return FR_OK;
}

}  // namespace

// For measurements: one-token steps launched after this call record their CTAs' timestamps in `trace`
// ([cta][8] 64-bit words, cta = (sequence * kv heads + kv head) * grid.x + block; null switches it off).
static unsigned long long* attention_trace = nullptr;
FR_EXPORT int attention_mma_set_trace(unsigned long long* trace) {
    attention_trace = trace;
    return FR_OK;
}

// How many clusters of `size` CTAs (the splits of one sequence and kv head in a one-token step) run at once on
// the current device, for head size hd; 0 if unknown.
FR_EXPORT int attention_mma_clusters_at_once(int hd, int size) {
    switch (hd) {
        case 16: return clusters_at_once<16>(size);
        case 32: return clusters_at_once<32>(size);
        case 48: return clusters_at_once<48>(size);
        case 64: return clusters_at_once<64>(size);
        case 80: return clusters_at_once<80>(size);
        case 96: return clusters_at_once<96>(size);
        case 112: return clusters_at_once<112>(size);
        case 128: return clusters_at_once<128>(size);
        default: return 0;
    }
}

FR_EXPORT int attention_mma_supports(int hd, int page) { return hd % 16 == 0 && hd >= 16 && hd <= 128 && page == BLOCK_N; }

// q: rows of q_stride bf16 (head h at h * hd); out [rows][nq * hd]; pools [pool_pages][64][nkv][hd] bf16.
// seq_start/seq_qlen/seq_pos0: per sequence, its first row, its rows in this step, the position of its first row.
// seq_live (may be null): indexed by a sequence's first row; negative marks a sequence that has ended.
// max_q_len: the longest seq_qlen (sizes the grid).  keys_mode: 1 for one-token steps.  splits > 1 needs
// scratch of rows * nq * splits * (hd + 2) floats.  counters (may be null): n_counters zeroed ints; with them the
// splits of a one-token step are merged inside the kernel, without them by a second kernel.  status: a device word
// that receives a code (21 the copying warp, 22 a computing warp) if a bounded wait of a one-token step gives up.
FR_EXPORT int attention_mma(const void* q, int q_stride, void* out, const void* k_pool, const void* v_pool, int pool_pages,
                            const int* block_table, int table_width, int page, const int* seq_start,
                            const int* seq_qlen, const int* seq_pos0, const int* seq_live, int n_seqs, int rows,
                            int max_q_len, int nq, int nkv, int hd, int window, float scale, int keys_mode, int splits,
                            float* scratch, int* counters, int n_counters, int* status, cudaStream_t stream) {
    if (n_seqs <= 0 || rows <= 0) return FR_OK;
    if (!attention_mma_supports(hd, page)) FR_REFUSE("attention_mma: head size %d / page %d is not built", hd, page);
    if (nkv <= 0 || nq % nkv != 0) FR_REFUSE("attention: %d heads cannot share %d key/value heads", nq, nkv);
    if (splits < 1 || splits > 4096) FR_REFUSE("attention_mma: %d splits", splits);
    if (splits > 8 && scratch == nullptr) FR_REFUSE("attention_mma: more than 8 splits need a scratch buffer");
    if (keys_mode && status == nullptr) FR_REFUSE("attention_mma: one-token steps need a status word");
    if (n_seqs > 65535 || nkv > 65535) FR_REFUSE("attention_mma: %d sequences x %d kv heads exceed the grid", n_seqs, nkv);
    MmaArgs p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.k_pool = (const bf16*)k_pool; p.v_pool = (const bf16*)v_pool;
    p.block_table = block_table; p.seq_start = seq_start; p.seq_qlen = seq_qlen; p.seq_pos0 = seq_pos0;
    p.seq_live = seq_live; p.part = scratch; p.counters = keys_mode ? counters : nullptr;
    p.cluster = keys_mode && splits >= 2 && splits <= 8 && use_clusters();
    p.q_stride = q_stride; p.table_width = table_width; p.nq = nq;
    p.nkv = nkv; p.window = window; p.splits = splits; p.scale_log2 = scale * LOG2E;
    p.trace = keys_mode ? attention_trace : nullptr;
    p.status = status;
    p.pool_rows = pool_pages * BLOCK_N;
    const int G = nq / nkv;
    const int rows_cta = keys_mode ? 16 : 64;
    const int tiles = (max_q_len * G + rows_cta - 1) / rows_cta;
    if (p.counters != nullptr && ((long long)n_seqs * nkv * tiles > n_counters || splits > 64))
        p.counters = nullptr;                          // the merge kernel instead
    dim3 grid(tiles * splits, nkv, n_seqs);
    CUtensorMap mk = {}, mv = {};
    if (keys_mode) {
        if (pool_pages <= 0 || ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15))
            FR_REFUSE("attention_mma: one-token steps need the pools' size and 16-byte aligned pools");
        int rc_map = pool_map(&mk, k_pool, pool_pages, nkv, hd);
        if (rc_map) return rc_map;
        rc_map = pool_map(&mv, v_pool, pool_pages, nkv, hd);
        if (rc_map) return rc_map;
    }
    int rc = keys_mode ? launch_hd<true>(hd, mk, mv, p, grid, stream) : launch_hd<false>(hd, mk, mv, p, grid, stream);
    if (rc) return rc;
    if (splits > 1 && p.counters == nullptr && !p.cluster) {
        MergeArgs mp{scratch, out, rows, nq, hd, splits};
        FR_CUDA(fr_launch(attention_merge_kernel<bf16>, dim3((rows * nq + 3) / 4), dim3(128), 0, stream, mp));
        FR_CHECK_LAUNCH("attention merge");
    }
    return FR_OK;
}
