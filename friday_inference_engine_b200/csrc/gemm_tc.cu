// bf16 matrix product on the 5th-generation tensor cores (sm_100a):
//
//     out[m][n] = sum_k x[m][k] * w[n][k]  (+ bias[n]) (+ residual[m][n]),  fp32 sums
//
// x: activations [rows][k], w: projection weights [out][in]; both are row-major with k
// innermost ("K-major"), which is the layout tcgen05.mma takes for both operands, so
// nothing is transposed or copied.  One persistent kernel per launch:
//
//   warp 0      TMA producer: cp.async.bulk.tensor.2d loads of 64-element (128-byte) wide
//               k-slices of both operands into a ring of shared-memory stages, 128-byte
//               swizzle, completion on an mbarrier per stage.  No cluster multicast.
//   warp 1      allocates tensor memory, then one lane issues tcgen05.mma
//               (cta_group::1, kind::f16, M=128, N=BN, K=16) from shared-memory
//               descriptors; tcgen05.commit hands stages back to the producer and
//               accumulators on to the epilogue.
//   warps 2-5   epilogue: tcgen05.ld of the fp32 accumulators (TMEM lanes = rows of the
//               tile), bias, residual, rounding, stores.  Two accumulator buffers in
//               TMEM let the epilogue of one tile overlap the products of the next.
//
// The operand that feeds the M side of the instruction ("P", tiles of 128 rows) and the
// one that feeds its N side ("Q", tiles of BN rows) are chosen by the launcher:
//   many rows (prompts):   P = x, Q = w, BN = 128 ... 256 in steps of 16 (the widest
//                          kernel instance takes the width as a number), chosen so that
//                          the tiles fill whole waves; with more than 128 rows and at
//                          least 256 columns the tiles are 256 rows high and run on
//                          pairs of SMs (gemm_tc_pair.cuh, cta_group::2);
//   few rows (decoding):   P = w, Q = x, BN = 16/32/64 >= rows (up to 64 rows): every
//                          weight is streamed once at full width, the handful of
//                          activations ride along, and the epilogue writes the tile
//                          transposed: the sums go through shared memory as
//                          [rows][128 columns] floats, then every thread finishes pieces
//                          of 8 consecutive columns of one row with 16-byte accesses.
// In that transposed epilogue more can ride along (gemm_tc_fusion.h): the RMSNorm of
// the input finished (a factor per row), the RMSNorm of the output begun, and rotary
// encoding with the write of keys and values into the cache.  What it reads besides
// the sums is fetched while the products run.
// When a shape has fewer tiles than the GPU has SMs (decoding against a [4608 x 3584]
// matrix is 36 tiles), k is cut into `splits` ranges; each CTA writes its partial tile to
// a scratch buffer, and the CTA that arrives last for a tile (a counter per tile) sums
// the partials in split order and runs the epilogue.  The sum order is fixed, so results
// do not depend on which CTA came last.  Tiles of 32 or 64 rows are finished by all the
// CTAs of the tile instead, 16 rows each, once every partial tile is written (they wait
// for the tile's counter, with a time limit): one CTA alone took 24 us for such a tile.
//
// Replaces the reference's int8 mma.sync GEMM (prefill_kernels.cu:173-327) and its dp4a
// GEMVs (hpc_k_quants.cu:445-681), with the same epilogue contract (bias, then
// residual, in place allowed: prefill_kernels.cu:156-171, hpc_k_quants.cu:404-437).
//
// Every wait on an mbarrier is bounded: after about two seconds the waiting thread
// records a code in `status` and all roles leave their loops, free TMEM and return.
#include <cuda.h>

#include "common.cuh"
#include <atomic>
#include <mutex>
#include <unordered_map>
#include "tc_common.cuh"

FR_EXPORT const char* gemm_tc_last_error() { return fr_error_text; }

#include "gemm_tc_fusion.h"

namespace {

using namespace tc;
constexpr int THREADS = 192;
constexpr int SIDE_BYTES = 3 * TILE_P * 4 + 3 * 64 * 4 + 64 * 8;      // row factors and what the epilogue of narrow tiles prefetches

// Dynamic shared memory of a kernel instance: the ring of stages (1 KB alignment slack), barriers, the TMEM
// slot and flags (64 bytes), the row factors, and the staging tile of narrow instances.
template <int BN, int STAGES>
constexpr int smem_bytes() {
    return STAGES * (P_BYTES + BN * TILE_K * 2) + 1024 + (2 * STAGES + 4) * 8 + 64 + SIDE_BYTES +
           (BN <= 32 ? BN * TILE_P * 4 : BN == 64 || BN == 128 ? 16 * TILE_P * 4 : BN * 4) + (BN <= 64 ? 16 * 64 * 8 : 0);
}

struct GemmParams {
    GemmFusion f;
    void* out;
    const void* bias;
    const void* residual;
    float* ws;          // [tiles][splits][BN/16][128][16] partial tiles when splits > 1
    int* counters;      // [tiles], zero between launches
    int* status;        // 0, or a code when a wait gave up
    int p_rows, q_rows, ldo, out_dtype, bias_dtype, swapped;
    int bn;             // rows of Q per tile: the kernel's BN, or any multiple of 16 below it in the widest instance
    int act;            // 1: the product's columns are (gate, up) pairs; out gets silu(gate) * up, half as wide
    int tiles_p, tiles_q, splits, kb_total, kb_per;
    // Work decomposition.  The first dp_tiles tiles are cut into `splits` equal k ranges each and dealt out round
    // robin (splits = 1: whole tiles).  The remaining sk_tiles tiles ("stream-k"): their k blocks, laid end to end,
    // are cut into one contiguous run of sk_units per CTA, so that a last, partial wave of tiles keeps every SM busy.
    int dp_tiles, sk_tiles, sk_units;
    // Tiles wider than 16 rows whose k is split: instead of the last CTA to arrive finishing the whole tile, every
    // CTA of the tile waits until all partial tiles are written and finishes a share of the tile's rows (16 at a
    // time).  Needs all CTAs of a tile on the device at once (grid = tiles * splits, no more than there are SMs), and a
    // second counter per tile (at counters[tiles + tile]) that tells the last CTA to leave.
    int shared_finish;
};

struct Item {
    int tile;        // which tile
    int kb0, kb1;    // its k blocks [kb0, kb1)
    int nseg;        // items that share the tile (1: this item has it alone and writes the output itself)
    int part;        // slot of this item's partial tile in the scratch buffer (nseg > 1)
    int first;       // stream-k: the first CTA that contributes to the tile (their slots follow from that)
};

// The items of one CTA, in the order in which all three roles walk them.
struct Work {
    const GemmParams& p;
    int cta, grid, i, u, u_end;
    __device__ Work(const GemmParams& p_, int cta_, int grid_) : p(p_), cta(cta_), grid(grid_), i(0) {
        const int total = p.sk_tiles * p.kb_total;
        u = min(cta * p.sk_units, total);
        u_end = min(u + p.sk_units, total);
    }
    __device__ bool next(Item& it) {
        const int w = cta + i * grid;
        if (w < p.dp_tiles * p.splits) {
            ++i;
            it.tile = w / p.splits;
            const int split = w - it.tile * p.splits;
            it.kb0 = split * p.kb_per;
            it.kb1 = min(it.kb0 + p.kb_per, p.kb_total);
            it.nseg = p.splits;
            it.part = w;
            it.first = -1;
            return true;
        }
        if (u >= u_end) return false;
        const int t = u / p.kb_total;                      // tile among the stream-k tiles
        it.tile = p.dp_tiles + t;
        it.kb0 = u - t * p.kb_total;
        it.kb1 = min(p.kb_total, it.kb0 + (u_end - u));
        u += it.kb1 - it.kb0;
        it.first = (t * p.kb_total) / p.sk_units;
        it.nseg = ((t + 1) * p.kb_total - 1) / p.sk_units - it.first + 1;
        it.part = sk_slot(cta, t);
        return true;
    }
    // A CTA writes at most two partial tiles: of the first tile of its run (slot 0) and of a later one (slot 1).
    __device__ int sk_slot(int c, int t) const { return 2 * c + (t > (c * p.sk_units) / p.kb_total ? 1 : 0); }
    __device__ int contributor(const Item& it, int s) const {          // slot of the s-th partial of the tile
        return it.first < 0 ? it.tile * p.splits + s : sk_slot(it.first + s, it.tile - p.dp_tiles);
    }
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ void mark(const GemmParams& p, int point) {
    if (p.f.trace != nullptr) p.f.trace[(size_t)blockIdx.x * 16 + point] = global_ns();
}

// Rows on the M side, the RMSNorm of the output begun: 16 whole columns gj0.. of row gi (the launcher has seen to
// n % 16 == 0 and 16-byte aligned rows): bias, residual, rounding, store; then the rounded values' squares into ss and,
// times the norm's weights g16[0..15], into norm_out.  pre_added: bias and residual are in v already.
__device__ __forceinline__ void finish16_begin_norm(const GemmParams& p, const float* g16, int gi, int gj0, float (&v)[16],
                                                    float& ss, bool pre_added = false) {
    if (gi >= p.p_rows || gj0 >= p.q_rows) return;
    const size_t base = (size_t)gi * p.ldo + gj0;
    if (p.bias != nullptr && !pre_added)
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] += bias_at(p, gj0 + j);
    if (p.residual != nullptr && !pre_added) {
        const uint4* rp = (const uint4*)((const __nv_bfloat16*)p.residual + base);
        const uint4 r0 = rp[0], r1 = rp[1];
        const uint32_t rw[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[2 * j] += __uint_as_float(rw[j] << 16);
            v[2 * j + 1] += __uint_as_float(rw[j] & 0xffff0000u);
        }
    }
    uint32_t w[8], h[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        w[j] = pack2(v[2 * j], v[2 * j + 1]);
        const float x0 = __uint_as_float(w[j] << 16), x1 = __uint_as_float(w[j] & 0xffff0000u);
        ss += x0 * x0;
        ss += x1 * x1;
        h[j] = pack2(x0 * g16[2 * j], x1 * g16[2 * j + 1]);
    }
    uint4* o = (uint4*)((__nv_bfloat16*)p.out + base);
    o[0] = make_uint4(w[0], w[1], w[2], w[3]);
    o[1] = make_uint4(w[4], w[5], w[6], w[7]);
    uint4* ho = (uint4*)((__nv_bfloat16*)p.f.norm_out + base);
    ho[0] = make_uint4(h[0], h[1], h[2], h[3]);
    ho[1] = make_uint4(h[4], h[5], h[6], h[7]);
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
               const GemmParams p) {
    // The widest instance takes any tile width up to its own (a multiple of 16): strides in shared and tensor memory
    // stay those of the full width, the boxes of the loads, the instruction and the loops follow p.bn.
    const int bn = BN == 256 ? p.bn : BN;
    constexpr int Q_BYTES = BN * TILE_K * 2;
    constexpr int STAGE_BYTES = P_BYTES + Q_BYTES;
    constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);
    // bars: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    int* flags = (int*)(tmem_slot + 1);      // flags[0]: this CTA came last for the tile (split-k)
    // One factor per row of the step in this tile (the deferred RMSNorm of the input).
    float* s_scale = (float*)((uint8_t*)(bars + 2 * STAGES + 4) + 64);      // [128]
    // What the epilogue of a narrow tile reads per tile, fetched early: bias and norm weights of the tile's columns,
    // rotary denominators, each row's sequence, position and cache row, the rotation's (cos, sin) per row and pair.
    float* s_g = s_scale + TILE_P;                                           // [128]
    float* s_bias = s_g + TILE_P;                                            // [128]
    float* s_den = s_bias + TILE_P;                                          // [64]
    int* s_seq = (int*)(s_den + 64);                                         // [64]
    int* s_pos = s_seq + 64;                                                 // [64]
    long long* s_crow = (long long*)(s_pos + 64);                            // [64]
    // Narrow tiles (the swapped orientation) write their output transposed: the sums of [BN rows][128 columns]
    // go through this buffer so that global memory sees 16-byte pieces of whole rows.
    // (64- and 128-wide tiles of the swapped orientation go through a window of 16 of their rows at a time: 24 KB less
    // than a whole 64-wide tile, one more stage of the ring)
    constexpr int W_ROWS = BN <= 32 ? BN : 16;
    constexpr int T_BYTES = BN <= 64 || BN == 128 ? W_ROWS * TILE_P * 4 : 0;
    uint8_t* s_tile = (uint8_t*)s_scale + SIDE_BYTES;
    float2* s_cs = (float2*)(s_tile + T_BYTES);                              // [16][64]: the rotation's (cos, sin) of the 16 rows being finished
    float* s_gw = (float*)s_tile;                                            // [BN] norm weights of the columns of a tile with rows on M
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t accf0 = smem_u32(bars + 2 * STAGES), acce0 = smem_u32(bars + 2 * STAGES + 2);

    if (threadIdx.x == 0) {
        mark(p, 0);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(accf0 + 8 * a, 1);
            mbar_init(acce0 + 8 * a, 4);
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
    if (threadIdx.x == 0) {
        fr_pdl_launch();                       // the next kernel may be scheduled; it waits for this one itself
        mark(p, 1);
    }

    if (warp == 0) {
        if (elect_one()) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_p) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
            // The k-slices this CTA will load, in order: (work item, k block).
            struct Walk {
                Work work;
                Item item;
                int kb, p_blk, q_blk;
                bool live;
                __device__ Walk(const GemmParams& pp, int cta, int grid) : work(pp, cta, grid), live(true) { open(pp); }
                __device__ void open(const GemmParams& pp) {
                    live = work.next(item);
                    if (!live) return;
                    q_blk = item.tile / pp.tiles_p;
                    p_blk = item.tile - q_blk * pp.tiles_p;
                    kb = item.kb0;
                }
                __device__ void step(const GemmParams& pp) {
                    if (++kb >= item.kb1) open(pp);
                }
            };
            // The weights do not depend on the kernel before this one; the activations do.  Fill the ring with
            // weight slices first, then wait for the predecessor, then add the activation slices.
            const uint32_t stage_tx = P_BYTES + bn * TILE_K * 2;       // bytes that land in a stage
            const CUtensorMap* map_w = p.swapped ? &map_p : &map_q;
            const CUtensorMap* map_x = p.swapped ? &map_q : &map_p;
            const uint32_t off_w = p.swapped ? 0 : P_BYTES, off_x = p.swapped ? P_BYTES : 0;
            Walk head(p, blockIdx.x, gridDim.x);
            Walk ahead(p, blockIdx.x, gridDim.x);
            int early = 0;
            for (; early < STAGES && ahead.live; ++early, ahead.step(p)) {
                mbar_expect_tx(full0 + 8 * early, stage_tx);
                tma_load_2d(smem_u32(smem + early * STAGE_BYTES) + off_w, map_w, ahead.kb * TILE_K,
                            p.swapped ? ahead.p_blk * TILE_P : ahead.q_blk * bn, full0 + 8 * early);
            }
            mark(p, 2);
            fr_pdl_wait();
            mark(p, 3);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (; head.live && ok; head.step(p)) {
                const uint32_t dst = smem_u32(smem + stage * STAGE_BYTES);
                if (early > 0) {
                    --early;                                 // the weight slice of this stage is already on its way
                } else {
                    if (!(ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, p.status, 1))) break;
                    mbar_expect_tx(full0 + 8 * stage, stage_tx);
                    tma_load_2d(dst + off_w, map_w, head.kb * TILE_K, p.swapped ? head.p_blk * TILE_P : head.q_blk * bn,
                                full0 + 8 * stage);
                }
                tma_load_2d(dst + off_x, map_x, head.kb * TILE_K, p.swapped ? head.q_blk * bn : head.p_blk * TILE_P,
                            full0 + 8 * stage);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            fr_pdl_wait();
            const uint32_t idesc = instr_desc(TILE_P, bn);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int it = 0;
            Work work(p, blockIdx.x, gridDim.x);
            Item item;
            for (; ok && work.next(item); ++it) {
                const int kb0 = item.kb0, kb1 = item.kb1;
                const int a = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!(ok = mbar_wait(acce0 + 8 * a, acc_phase ^ 1, p.status, 2))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + a * BN;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!(ok = mbar_wait(full0 + 8 * stage, phase, p.status, 3))) break;
                    if (it == 0 && kb == kb0) mark(p, 4);
                    tc_fence_after();
                    const uint32_t pa = smem_u32(smem + stage * STAGE_BYTES);
                    const uint64_t da = smem_desc(pa), db = smem_desc(pa + P_BYTES);
#pragma unroll
                    for (int k = 0; k < TILE_K / UMMA_K; ++k)
                        tc_mma(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    tc_commit(empty0 + 8 * stage);        // the stage is free once these products are done
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) tc_commit(accf0 + 8 * a);         // the accumulator is complete
            }
            mark(p, 5);
        }
    } else {
        const int quarter = warp & 3;                      // TMEM lanes this warp may read: 32*quarter ..
        const int i_local = quarter * 32 + lane;
        const int et = threadIdx.x - 64;                   // 0..127 among the epilogue threads
        fr_pdl_wait();
        bool ok = true;
        int it = 0;
        const GemmFusion& f = p.f;
        // Narrow tiles of the swapped orientation are written transposed.  Their sums go through s_sum as
        // [rows of the step][128 columns] floats; then every thread finishes pieces of 8 consecutive columns of one
        // row (bias, residual, rounding, and the fused work) with 16-byte accesses to global memory.
        const bool bf16_out = p.out_dtype == FR_BF16;
        const bool can_stage = T_BYTES > 0 && p.swapped && (p.ldo % 8) == 0 &&
                               (((uintptr_t)p.out | (uintptr_t)p.residual) & 15) == 0 && (bf16_out || p.residual == nullptr);
        const bool rope = f.row_pos != nullptr;            // the launcher grants it to tiles of up to 64 rows
        float* s_sum = (float*)s_tile;
        constexpr int ITEMS = 2;                           // pieces per thread of 16 rows: 16 * 16 pieces over 128 threads
        uint4 res[ITEMS];                                  // this thread's pieces of the residual rows being finished
        if (rope && f.denom != nullptr && et < (f.rot >> 1)) s_den[et] = f.denom[et];
        // What a staged tile's epilogue reads besides the sums is fetched as soon as the tile is known, while the
        // products are still running: bias and norm weights of the tile's columns, the residual pieces, each row's
        // sequence, position and cache row, and the rotation's cosines and sines.  What remains after the last product
        // is one trip to memory for split-k's partial sums, arithmetic, and stores.
        // this thread's pieces of the residual rows t_lo .. t_lo + t_cnt - 1 of the tile
        auto load_res = [&](int p_blk, int q_blk, int t_lo, int t_cnt) {
            if (p.residual == nullptr) return;
#pragma unroll
            for (int k = 0; k < ITEMS; ++k) {
                const int idx = et + 128 * k;
                if (idx < t_cnt * 16)
                    res[k] = __ldcg((const uint4*)((const __nv_bfloat16*)p.residual + (size_t)(q_blk * bn + t_lo + (idx >> 4)) * p.ldo +
                                                   (size_t)p_blk * TILE_P + (idx & 15) * 8));
            }
        };
        // r_lo, r_cnt: the rows of the tile whose residual pieces this CTA will need first (16-wide tiles)
        auto prefetch_tile = [&](int p_blk, int q_blk, int r_lo, int r_cnt) {
            const int nt = min(bn, p.q_rows - q_blk * bn);
            s_bias[et] = p.bias != nullptr ? bias_at(p, p_blk * TILE_P + et) : 0.f;
            if (f.norm_out != nullptr)
                s_g[et] = f.norm_w_dtype == FR_F32 ? ((const float*)f.norm_w)[p_blk * TILE_P + et]
                                                   : __bfloat162float(((const __nv_bfloat16*)f.norm_w)[p_blk * TILE_P + et]);
            if (BN == 16) load_res(p_blk, q_blk, r_lo, min(r_cnt, nt - r_lo));   // wider tiles fetch them 16 rows at a time, when they finish them
            if (rope && et < nt) {
                const int row = q_blk * bn + et;
                const int seq = f.row_seq[row], pos = f.row_pos[row];
                s_seq[et] = seq;
                s_pos[et] = pos;
                long long crow = -1;
                if (seq >= 0 && f.k_pool != nullptr) {
                    const int pg = f.table[(size_t)seq * f.table_width + pos / f.page];
                    crow = ((long long)pg * f.page + pos % f.page) * f.nkv * f.hd;
                }
                s_crow[et] = crow;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (BN == 16 && rope && f.denom != nullptr) {       // wider tiles make them 16 rows at a time, when they finish them
                const int half = f.rot >> 1;
                for (int idx = et; idx < nt * half; idx += 128) {
                    const int token = idx / half, i = idx - token * half;
                    float sn = 0.f, cs = 1.f;
                    if (s_seq[token] >= 0) sincosf(__fdiv_rn((float)s_pos[token], s_den[i]), &sn, &cs);
                    s_cs[token * 64 + i] = make_float2(cs, sn);
                }
            }
        };
        // 16 rows of the step for this thread's column: into the transposed tile.
        auto put16 = [&](int c, const float (&v)[16]) {
#pragma unroll
            for (int j = 0; j < 16; ++j) s_sum[((c * 16 + j) & (W_ROWS - 1)) * TILE_P + i_local] = v[j];
        };
        // bias and residual added to 8 sums of one row; the values as they will be stored (bf16: rounded)
        auto load_piece = [&](int token, int f0, float (&x)[8]) {
            const float* at = s_sum + (token & (W_ROWS - 1)) * TILE_P + f0;
            const float4 a0 = *(const float4*)at, a1 = *(const float4*)(at + 4);
            const float4 b0 = *(const float4*)(s_bias + f0), b1 = *(const float4*)(s_bias + f0 + 4);
            x[0] = a0.x + b0.x; x[1] = a0.y + b0.y; x[2] = a0.z + b0.z; x[3] = a0.w + b0.w;
            x[4] = a1.x + b1.x; x[5] = a1.y + b1.y; x[6] = a1.z + b1.z; x[7] = a1.w + b1.w;
        };
        auto round8 = [&](const float (&x)[8]) {
            uint4 w;
            w.x = pack2(x[0], x[1]); w.y = pack2(x[2], x[3]); w.z = pack2(x[4], x[5]); w.w = pack2(x[6], x[7]);
            return w;
        };
        // The gated epilogue on a staged tile: the tile's 128 columns are 64 (gate, up) pairs; a thread turns 16 sums of
        // one row into 8 values silu(gate) * up and stores them as one 16-byte piece (8 pieces per row, 16 rows a time).
        auto finish_rows_gated = [&](int p_blk, int q_blk, int t_lo, int t_cnt) {
            if (et >= t_cnt * 8) return;
            const int token = t_lo + (et >> 3), f0 = (et & 7) * 16;
            const float* src = s_sum + (token & (W_ROWS - 1)) * TILE_P + f0;
            float x[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 a = *(const float4*)(src + 4 * j);
                x[2 * j] = silu_mul(a.x, a.y);
                x[2 * j + 1] = silu_mul(a.z, a.w);
            }
            __nv_bfloat16* out_at = (__nv_bfloat16*)p.out + (size_t)(q_blk * bn + token) * p.ldo + ((p_blk * TILE_P + f0) >> 1);
            *(uint4*)out_at = round8(x);
        };
        auto finish_rows = [&](int p_blk, int q_blk, int t_lo, int t_cnt) {     // rows t_lo .. t_lo + t_cnt - 1 of the tile
            if (p.act) {
                finish_rows_gated(p_blk, q_blk, t_lo, t_cnt);
                return;
            }
            const int half = f.rot >> 1;
#pragma unroll
            for (int k = 0; k < ITEMS; ++k) {
                if (k * 128 >= t_cnt * 16) break;
                const int idx = k * 128 + et, token = t_lo + (idx >> 4), f0 = (idx & 15) * 8;
                const bool active = idx < t_cnt * 16;
                const int row = q_blk * bn + token, col = p_blk * TILE_P + f0;
                float ss = 0.f;
                if (active) {
                    float x[8];
                    load_piece(token, f0, x);
                    if (!bf16_out) {
                        float4* dst = (float4*)((float*)p.out + (size_t)row * p.ldo + col);
                        dst[0] = make_float4(x[0], x[1], x[2], x[3]);
                        dst[1] = make_float4(x[4], x[5], x[6], x[7]);
                    } else {
                        if (p.residual != nullptr) {
                            const uint32_t r[4] = {res[k].x, res[k].y, res[k].z, res[k].w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                x[2 * j] += __uint_as_float(r[j] << 16);
                                x[2 * j + 1] += __uint_as_float(r[j] & 0xffff0000u);
                            }
                        }
                        __nv_bfloat16* out_at = (__nv_bfloat16*)p.out + (size_t)row * p.ldo + col;
                        uint4 w = round8(x);
                        if (rope) {
                            // heads never straddle tiles; f_in: the piece's first column within its head
                            const int h = col / f.hd, f_in = col - h * f.hd;
                            const long long crow = s_crow[token];
                            __nv_bfloat16* cache_at = nullptr;
                            if (crow >= 0 && h >= f.nq)
                                cache_at = (h < f.nq + f.nkv ? (__nv_bfloat16*)f.k_pool + (size_t)(h - f.nq) * f.hd
                                                             : (__nv_bfloat16*)f.v_pool + (size_t)(h - f.nq - f.nkv) * f.hd) + crow + f_in;
                            if (f.denom != nullptr && h < f.nq + f.nkv && f_in < f.rot && s_seq[token] >= 0) {
                                if (f_in < half) {
                                    // this piece and its partner `half` columns on, rotated together
                                    float y[8];
                                    load_piece(token, f0 + half, y);
                                    const uint4 wy = round8(y);
                                    const uint32_t lo[4] = {w.x, w.y, w.z, w.w}, hi[4] = {wy.x, wy.y, wy.z, wy.w};
                                    float ra[8], rb[8];
#pragma unroll
                                    for (int j = 0; j < 8; ++j) {
                                        const float a = __uint_as_float(j & 1 ? lo[j >> 1] & 0xffff0000u : lo[j >> 1] << 16);
                                        const float b = __uint_as_float(j & 1 ? hi[j >> 1] & 0xffff0000u : hi[j >> 1] << 16);
                                        const float2 cs = s_cs[(token - (BN == 16 ? 0 : t_lo)) * 64 + f_in + j];
                                        fr_rotate(a, b, cs.x, cs.y, ra[j], rb[j]);
                                    }
                                    const uint4 wa = round8(ra), wb = round8(rb);
                                    *(uint4*)out_at = wa;
                                    *(uint4*)(out_at + half) = wb;
                                    if (cache_at != nullptr) {
                                        *(uint4*)cache_at = wa;
                                        *(uint4*)(cache_at + half) = wb;
                                    }
                                }
                            } else {
                                *(uint4*)out_at = w;
                                if (cache_at != nullptr) *(uint4*)cache_at = w;
                            }
                        } else {
                            *(uint4*)out_at = w;
                            if (f.norm_out != nullptr) {
                                // the RMSNorm that follows, begun: g (*) x rounded, and this piece's share of the row's
                                // sum of squares (sixteen lanes per row, summed in a fixed order below)
                                const uint32_t r[4] = {w.x, w.y, w.z, w.w};
                                float hx[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    const float xr = __uint_as_float(j & 1 ? r[j >> 1] & 0xffff0000u : r[j >> 1] << 16);
                                    ss += xr * xr;
                                    hx[j] = xr * s_g[f0 + j];
                                }
                                *(uint4*)((__nv_bfloat16*)f.norm_out + (size_t)row * p.ldo + col) = round8(hx);
                            }
                        }
                    }
                }
                if (f.norm_out != nullptr) {
#pragma unroll
                    for (int o = 1; o < 16; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    if (active && f0 == 0) f.out_ssq[(size_t)p_blk * p.q_rows + row] = ss;
                }
            }
        };
        // The factors 1 / sqrt(mean x^2 + eps) of the rows of the step that this tile covers.
        int scale_blk = -1;
        auto load_scale = [&](int blk) {
            if (f.in_ssq == nullptr || blk == scale_blk) return;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int rows = p.swapped ? p.q_rows : p.p_rows, per = p.swapped ? bn : TILE_P;
            if (et < per) {
                const int row = blk * per + et;
                float ss = 0.f;
                if (row < rows)
                    for (int t = 0; t < f.in_parts; ++t) ss += __ldcg(f.in_ssq + (size_t)t * rows + row);
                s_scale[et] = 1.0f / sqrtf(ss / f.in_width + f.in_eps);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            scale_blk = blk;
        };
        auto scale16 = [&](int c, float (&v)[16]) {
            if (f.in_ssq == nullptr) return;
            if (p.swapped) {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] *= s_scale[(c * 16 + j) & (TILE_P - 1)];
            } else {
                const float r = s_scale[i_local];
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] *= r;
            }
        };
        auto finish16_norm = [&](int q_blk, int gi, int gj0, float (&v)[16], float& ss) {
            finish16_begin_norm(p, s_gw + (gj0 - q_blk * bn), gi, gj0, v, ss);
        };
        const bool norm_rows = f.norm_out != nullptr && !p.swapped;
        // Rows of a staged tile are finished 16 at a time (a chunk of the accumulator's columns): chunks c_begin,
        // c_begin + c_step, ...  With `summed` the chunk's sums are first gathered from the tile's partial tiles in the
        // scratch buffer (split-k); otherwise they lie in s_sum already.
        Work work(p, blockIdx.x, gridDim.x);
        Item item;
        auto finish_chunks = [&](int p_blk, int q_blk, int c_begin, int c_step, bool summed) {
            const int nt = min(bn, p.q_rows - q_blk * bn);
            const float* mine = p.ws + (size_t)i_local * 4;
#pragma unroll 1
            for (int c = c_begin; c * 16 < nt; c += c_step) {
                const int t_cnt = min(16, nt - c * 16);
                if (BN > 16) load_res(p_blk, q_blk, c * 16, t_cnt);
                if (summed) {
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0.f;
                    // five partial tiles at a time: all their loads are on their way before the first sum
                    for (int s0 = 0; s0 < item.nseg; s0 += 5) {
                        float4 x[5][4];
#pragma unroll
                        for (int s = 0; s < 5; ++s) {
                            if (s0 + s < item.nseg) {
                                const float* src = mine + (size_t)work.contributor(item, s0 + s) * TILE_P * bn + (size_t)c * TILE_P * 16;
#pragma unroll
                                for (int j = 0; j < 4; ++j) x[s][j] = __ldcg((const float4*)(src + (size_t)j * TILE_P * 4));
                            }
                        }
#pragma unroll
                        for (int s = 0; s < 5; ++s) {
                            if (s0 + s < item.nseg) {
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    v[4 * j] += x[s][j].x; v[4 * j + 1] += x[s][j].y;
                                    v[4 * j + 2] += x[s][j].z; v[4 * j + 3] += x[s][j].w;
                                }
                            }
                        }
                    }
                    if (et == 0) mark(p, 10);
                    scale16(c, v);
                    put16(c, v);
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (et == 0) mark(p, 11);
                }
                if (BN > 16 && rope && f.denom != nullptr) {
                    // the cosines and sines of these 16 rows (s_seq and s_pos were filled when the tile was taken)
                    const int half = f.rot >> 1;
                    for (int idx = et; idx < t_cnt * half; idx += 128) {
                        const int t = idx / half, i = idx - t * half;
                        float sn = 0.f, cs = 1.f;
                        if (s_seq[c * 16 + t] >= 0) sincosf(__fdiv_rn((float)s_pos[c * 16 + t], s_den[i]), &sn, &cs);
                        s_cs[t * 64 + i] = make_float2(cs, sn);
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                }
                finish_rows(p_blk, q_blk, c * 16, t_cnt);
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
        };
        // 16-wide tiles whose k-splits all finish a share of the tile: groups of 4 rows g_begin, g_begin + g_step, ...
        // (a thread's partial sums of 4 rows of its column are one 16-byte piece of a partial tile)
        auto finish_quarters = [&](int p_blk, int q_blk, int g_begin, int g_step) {
            const int nt = min(bn, p.q_rows - q_blk * bn);
            const float* mine = p.ws + (size_t)i_local * 4;
            bool first = true;
#pragma unroll 1
            for (int g = g_begin; g * 4 < nt; g += g_step) {
                const int t_cnt = min(4, nt - g * 4);
                if (!first) load_res(p_blk, q_blk, g * 4, t_cnt);      // the first group's pieces came when the tile was taken
                first = false;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int s0 = 0; s0 < item.nseg; s0 += 8) {
                    float4 x[8];
#pragma unroll
                    for (int sp = 0; sp < 8; ++sp)
                        if (s0 + sp < item.nseg)
                            x[sp] = __ldcg((const float4*)(mine + (size_t)work.contributor(item, s0 + sp) * TILE_P * bn + (size_t)g * TILE_P * 4));
#pragma unroll
                    for (int sp = 0; sp < 8; ++sp)
                        if (s0 + sp < item.nseg) { v.x += x[sp].x; v.y += x[sp].y; v.z += x[sp].z; v.w += x[sp].w; }
                }
                if (et == 0) mark(p, 10);
                if (f.in_ssq != nullptr) {
                    v.x *= s_scale[g * 4]; v.y *= s_scale[g * 4 + 1]; v.z *= s_scale[g * 4 + 2]; v.w *= s_scale[g * 4 + 3];
                }
                s_sum[(g * 4) * TILE_P + i_local] = v.x;
                s_sum[(g * 4 + 1) * TILE_P + i_local] = v.y;
                s_sum[(g * 4 + 2) * TILE_P + i_local] = v.z;
                s_sum[(g * 4 + 3) * TILE_P + i_local] = v.w;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (et == 0) mark(p, 11);
                finish_rows(p_blk, q_blk, g * 4, t_cnt);
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
        };
        for (; ok && work.next(item); ++it) {
            const int tile = item.tile;
            const int q_blk = tile / p.tiles_p, p_blk = tile - q_blk * p.tiles_p;
            const int a = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            const int gi = p_blk * TILE_P + i_local;
            const bool staged = can_stage && (p_blk + 1) * TILE_P <= p.p_rows;
            load_scale(p.swapped ? q_blk : p_blk);
            const bool quarters = BN == 16 && p.shared_finish && item.nseg > 1;      // this CTA finishes a share of the rows
            if (staged) prefetch_tile(p_blk, q_blk, quarters ? 4 * (item.part - tile * p.splits) : 0, quarters ? 4 : bn);
            float ss_row = 0.f;                            // rows-on-M with a norm begun: this row's sum of squares over the tile
            if (norm_rows) {
                asm volatile("bar.sync 1, 128;" ::: "memory");
                for (int i = et; i < bn; i += 128) {
                    const int col = q_blk * bn + i;
                    s_gw[i] = col >= p.q_rows ? 0.f : f.norm_w_dtype == FR_F32 ? ((const float*)f.norm_w)[col]
                                                                               : __bfloat162float(((const __nv_bfloat16*)f.norm_w)[col]);
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            if (!(ok = mbar_wait(accf0 + 8 * a, acc_phase, p.status, 4))) break;
            if (et == 0) mark(p, 6);
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + a * BN;
            // partial tiles are laid out [chunk of 16 columns][quarter of the chunk][row][4]: what a warp stores or
            // loads at a time is 512 bytes in one piece
            float* part = item.nseg > 1 ? p.ws + (size_t)item.part * TILE_P * bn + (size_t)i_local * 4 : nullptr;
#pragma unroll 1
            for (int c = 0; c < bn / 16; ++c) {
                uint32_t r[16];
                tc_ld16(taddr + c * 16, r);
                tc_ld_wait();
                float v[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
                if (part == nullptr) {
                    scale16(c, v);
                    if (staged) {
                        put16(c, v);
                        if (BN >= 64) {                    // the window holds these 16 rows only: finish them now
                            asm volatile("bar.sync 1, 128;" ::: "memory");
                            finish_chunks(p_blk, q_blk, c, BN, false);
                        }
                    }
                    else if (norm_rows) finish16_norm(q_blk, gi, q_blk * bn + c * 16, v, ss_row);
                    else finish16(p, gi, q_blk * bn + c * 16, v);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        *(float4*)(part + ((size_t)c * 4 + j) * TILE_P * 4) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce0 + 8 * a);     // the accumulator may be overwritten
            if (part == nullptr && staged && BN < 64) {
                asm volatile("bar.sync 1, 128;" ::: "memory");
                finish_chunks(p_blk, q_blk, 0, 1, false);
            }
            if (item.nseg > 1 && p.shared_finish && staged) {
                // The partial tile is written.  Tell the tile's other CTAs, wait for all of them (they all run: the
                // launcher saw to that), then finish every nseg-th group of 16 rows of the tile.
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (et == 0) {
                    __threadfence();
                    atomicAdd(p.counters + tile, 1);
                    const unsigned long long t_wait = global_ns();
                    bool all = false;
                    for (uint32_t spin = 1;; ++spin) {
                        if (*(volatile int*)(p.counters + tile) >= item.nseg) { all = true; break; }
                        if ((spin & 63u) == 0 && global_ns() - t_wait > WAIT_LIMIT_NS) break;
                    }
                    if (!all) atomicCAS(p.status, 0, 5);
                    __threadfence();
                    flags[0] = all;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (flags[0]) {
                    if (et == 0) mark(p, 8);
                    if (BN == 16) finish_quarters(p_blk, q_blk, item.part - tile * p.splits, item.nseg);
                    else finish_chunks(p_blk, q_blk, item.part - tile * p.splits, item.nseg, true);
                    if (et == 0) mark(p, 12);
                }
                // the last CTA to leave the tile makes its counters ready for the next launch
                if (et == 0 && atomicAdd(p.counters + p.dp_tiles + tile, 1) == item.nseg - 1) {
                    p.counters[tile] = 0;
                    p.counters[p.dp_tiles + tile] = 0;
                }
            } else if (item.nseg > 1) {
                // The partial tile is written; whoever adds the tile's last one sums them all (thread 0 of the epilogue
                // publishes for the CTA: the barrier before it orders the other threads' stores before its fence).
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (et == 0) {
                    __threadfence();
                    flags[0] = atomicAdd(p.counters + tile, 1) == item.nseg - 1;
                    __threadfence();
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (flags[0]) {
                    if (et == 0) mark(p, 8);
                    if (staged) {
                        finish_chunks(p_blk, q_blk, 0, 1, true);
                    } else {
                        const float* mine = p.ws + (size_t)i_local * 4;
#pragma unroll 1
                        for (int c = 0; c < bn / 16; ++c) {
                            float v[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) v[j] = 0.f;
#pragma unroll 2
                            for (int sp = 0; sp < item.nseg; ++sp) {
                                const float* src = mine + (size_t)work.contributor(item, sp) * TILE_P * bn + (size_t)c * TILE_P * 16;
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const float4 x = __ldcg((const float4*)(src + (size_t)j * TILE_P * 4));
                                    v[4 * j] += x.x; v[4 * j + 1] += x.y; v[4 * j + 2] += x.z; v[4 * j + 3] += x.w;
                                }
                            }
                            scale16(c, v);
                            if (norm_rows) finish16_norm(q_blk, gi, q_blk * bn + c * 16, v, ss_row);
                            else finish16(p, gi, q_blk * bn + c * 16, v);
                        }
                    }
                    if (et == 0) mark(p, 12);
                    if (et == 0) p.counters[tile] = 0;     // ready for the next launch
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            if (norm_rows && gi < p.p_rows && (item.nseg == 1 || flags[0])) f.out_ssq[(size_t)q_blk * p.p_rows + gi] = ss_row;
            if (et == 0) mark(p, 7);
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

}  // namespace

#include "gemm_tc_pair.cuh"

namespace {

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

// [rows][k] bf16, row stride ld elements; box = 64 elements of k by box_rows rows.
// A map depends on (address, shape, stride, box) only, and a model asks for the same few hundred over and over (its
// weights, and activations at the addresses its working memory repeats): the encoded maps are kept per thread.
struct MapKey {
    const void* base;
    int rows, k, ld, box_rows;
    bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && k == o.k && ld == o.ld && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& m) const {
        size_t h = (size_t)(uintptr_t)m.base * 0x9E3779B97F4A7C15ull;
        h ^= ((size_t)m.rows << 32 | (unsigned)m.k) * 0xC2B2AE3D27D4EB4Full;
        h ^= ((size_t)m.ld << 20 | (unsigned)m.box_rows) * 0x165667B19E3779F9ull;
        return h ^ (h >> 29);
    }
};

int encode_map(CUtensorMap* map, const void* base, int rows, int k, int ld, int box_rows);

int make_map(CUtensorMap* map, const void* base, int rows, int k, int ld, int box_rows) {
    static thread_local std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{base, rows, k, ld, box_rows};
    auto it = cache.find(key);
    if (it != cache.end()) {
        *map = it->second;
        return FR_OK;
    }
    const int rc = encode_map(map, base, rows, k, ld, box_rows);
    if (rc) return rc;
    if (cache.size() >= 8192) cache.clear();
    cache.emplace(key, *map);
    return FR_OK;
}

int encode_map(CUtensorMap* map, const void* base, int rows, int k, int ld, int box_rows) {
    EncodeTiled enc = encode_fn();
    if (enc == nullptr) FR_REFUSE("gemm_tc: the driver does not offer cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)TILE_K, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) FR_REFUSE("gemm_tc: cuTensorMapEncodeTiled failed with %d (rows %d, k %d, ld %d)", (int)r, rows, k, ld);
    return FR_OK;
}

// FRIDAY_STREAM_K=1 cuts a partial last wave of tiles along k over all SMs.  Off by default: measured at
// 2048 x 3584 x 3584 (224 tiles on 148 SMs) the merge of 128 x 256 partial tiles through global memory costs more
// (117 us) than the idle SMs of the last wave (59 us).
bool use_stream_k() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("FRIDAY_STREAM_K");
        v = (e != nullptr && e[0] == '1') ? 1 : 0;
    }
    return v != 0;
}

// FRIDAY_GEMM_EVEN_RUNS=1: products of few rows whose tiles fill several waves with a nearly empty last one run as
// equal runs of k blocks over all SMs.  Off by default: since the instructions of the copying and issuing threads
// became cheap (elect.sync), whole tiles are as fast or faster at every size measured (the head of 152,064 columns:
// 165.5 us against 168.2 us at 8 rows, 182.6 against 187.0 at 64, 203.3 against 213.0 at 128; the 14B shape's gate/up
// product: 48.9 against 50.2 us at 8 rows, 55.8 against 63.1 at 64).
bool use_even_runs() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("FRIDAY_GEMM_EVEN_RUNS");
        v = (e != nullptr && e[0] == '1') ? 1 : 0;
    }
    return v != 0;
}

// FRIDAY_GEMM_PAIR=0: products of many rows run on single SMs (128 x bn tiles) instead of pairs (256 x bn).
bool use_pair() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("FRIDAY_GEMM_PAIR");
        v = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

// Rows on the M side, more than one tile of 128 of them, wide outputs: pairs of SMs share 256 x bn tiles.
bool pair_shape(int m, int n, int swap, int sm_count) { return !swap && m > TILE_P && n >= 256 && sm_count >= 2 && use_pair(); }

// FRIDAY_GEMM_SHARED_FINISH=0: the last CTA of a tile to arrive always finishes the whole tile (for comparison).
bool use_shared_finish() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("FRIDAY_GEMM_SHARED_FINISH");
        v = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

// A kernel's shared-memory limit is a property of the function on one device: it is raised once per device, the
// devices that have it kept as bits of an atomic word (two host threads that both find the bit clear both set the
// attribute, which is harmless; neither launches before its own call has returned).
inline int current_device_bit(unsigned long long* bit) {
    int device = 0;
    FR_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= 64) FR_REFUSE("gemm_tc: device %d is outside the table of 64", device);
    *bit = 1ull << device;
    return FR_OK;
}

template <int BN, int STAGES>
int configure() {
    static std::atomic<unsigned long long> configured{0};
    unsigned long long bit = 0;
    const int rc = current_device_bit(&bit);
    if (rc) return rc;
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        FR_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     smem_bytes<BN, STAGES>()));
        configured.fetch_or(bit, std::memory_order_release);
    }
    return FR_OK;
}

template <int BN, int STAGES>
int launch(const CUtensorMap& mp, const CUtensorMap& mq, const GemmParams& p, int grid, cudaStream_t stream) {
    const int rc = configure<BN, STAGES>();
    if (rc) return rc;
    FR_CUDA(fr_launch(gemm_tc_kernel<BN, STAGES>, dim3(grid), dim3(THREADS), smem_bytes<BN, STAGES>(), stream, mp, mq, p));
    FR_CHECK_LAUNCH("gemm_tc");
    return FR_OK;
}

}  // namespace

// What the launcher would choose for a shape: fills plan[0..3] = {swapped, BN, splits, scratch floats needed}
// and plan[4] = counters needed.  bn / splits / swap < 0 let the heuristics decide.
FR_EXPORT int gemm_tc_plan(int m, int n, int k, int sm_count, int swap, int bn, int splits, long long* plan) {
    // Measured on B200 at the sizes of a 7B model (k = 3584 or 18944, n from 3584 to 152064):
    //  * up to 128 rows: weights on the M side, the rows as an N tile of 16, 32, 64 or 128; k split until the SMs are
    //    busy (at 64 rows: 16 / 15 / 35 us for the qkv, output and down products against 21 / 20 / 40 us the other
    //    way round; at 32 rows 13 / 12 / 31 against 21 / 20 / 39).  With the rows on the M side a CTA moves 16 KB of
    //    activations per k block whatever the number of rows, beside 4 KB of a narrow weight tile: at 96 rows the same
    //    three products took 15.4 / 14.9 / 42.7 us that way;
    //  * more rows: 128 x bn tiles, or 256 x bn tiles on pairs of SMs (wide outputs).
    const int kb_total = (k + TILE_K - 1) / TILE_K;
    if (swap < 0) swap = m <= 128 ? 1 : 0;
    const int q_rows = swap ? m : n, p_rows = swap ? n : m;
    const bool skinny = !swap && m <= TILE_P;
    if (bn <= 0) {
        if (swap) bn = q_rows <= 16 ? 16 : q_rows <= 32 ? 32 : q_rows <= 64 ? 64 : 128;
        else if (!skinny && q_rows >= 256) {
            // Many rows: 128 x bn tiles, bn a multiple of 16 from 128 to 256, chosen so that the tiles fill whole
            // waves of the SMs.  A tile costs about bn + 16 (its products, and an epilogue that is mostly hidden);
            // 2048 x 3584: 14 column tiles of 256 are 224 tiles, two waves at 76 %; 18 of 208 are 288, two at 97 %.
            // On pairs of SMs the tiles are 256 rows high and there are half as many units to fill.
            const bool pair = pair_shape(m, n, swap, sm_count);
            const long long tiles_p = pair ? (p_rows + 2 * TILE_P - 1) / (2 * TILE_P) : (p_rows + TILE_P - 1) / TILE_P;
            const long long units = pair ? sm_count / 2 : sm_count;
            long long best = -1;
            // (pairs of SMs also take narrower tiles; they pay where k is short and the wider tiles leave pairs idle:
            // 256 x 4608 x 3584 runs 36 tiles of 128 in 19.7 us and 72 of 64 in 17.6 us; long k is split instead)
            const int narrowest = pair && kb_total < 128 ? 64 : 128;
            for (int cand = 256; cand >= narrowest; cand -= 16) {
                const long long tiles = tiles_p * ((q_rows + cand - 1) / cand);
                const long long cost = ((tiles + units - 1) / units) * (cand + 16);
                if (best < 0 || cost < best) { best = cost; bn = cand; }
            }
        } else if (!skinny) bn = q_rows > 64 ? 128 : 64;
        else if (kb_total >= 128 && q_rows < 8192 && 2 * ((q_rows + 63) / 64) <= sm_count) bn = 64;   // long k, cut in two (96 x 3584 x 18944: 42.7 us; 128-wide tiles in four splits: 47.1 us)
        else if (q_rows >= 8192 || kb_total >= 128) bn = 128;
        else bn = (q_rows + 31) / 32 <= sm_count ? 32 : 64;
    }
    const int tiles = ((p_rows + TILE_P - 1) / TILE_P) * ((q_rows + bn - 1) / bn);
    if (splits <= 0) {
        splits = 1;
        if (tiles * 2 <= sm_count) {
            splits = sm_count / tiles;
            if (splits > kb_total / 4) splits = kb_total / 4;      // at least four k-slices per split
            if (skinny && splits > 4) splits = 4;                  // wide partial tiles are costly to merge
            // ... and with rows on the M side every partial tile is 128 or 256 rows high: a split pays only if it still
            // has 64 k blocks to itself (256 x 4608 x 3584: 19.7 us whole on 36 of 74 SM pairs, 23.2 us in two splits on
            // 72; 256 x 3584 x 18944: 72.5 us whole, 53.5 us in two)
            if (!swap && splits > kb_total / 64) splits = kb_total / 64;
            if (splits < 1) splits = 1;
        } else if (swap && bn <= 16 && tiles > sm_count) {
            // More tiles than SMs and a last wave that is partly empty (216 tiles on 148 SMs: the second wave costs as
            // much as the first for half the work): cutting k in two to four makes the waves shorter.  An item costs its
            // k blocks and about six more (filling the ring, partial tile, counter); the few rows of such a step keep
            // the sum of a tile's partial tiles cheap.
            const long long fixed = 6;
            long long best = (long long)((tiles + sm_count - 1) / sm_count) * (kb_total + fixed);
            for (int s = 2; s <= 4; ++s) {
                if (kb_total / s < 8) break;
                const long long cost = (long long)((tiles * s + sm_count - 1) / sm_count) * ((kb_total + s - 1) / s + fixed);
                if (cost * 20 < best * 19) { best = cost; splits = s; }
            }
        }
    }
    if (splits > kb_total) splits = kb_total;
    const int kb_per = (kb_total + splits - 1) / splits;
    splits = (kb_total + kb_per - 1) / kb_per;                     // no empty split
    plan[0] = swap; plan[1] = bn; plan[2] = splits;
    plan[3] = splits > 1 ? (long long)tiles * splits * TILE_P * bn : 0;
    plan[4] = splits > 1 ? tiles : 0;
    return FR_OK;
}

FR_EXPORT int gemm_tc_fused(const void* x, const void* w, void* out, int out_dtype, const void* bias, int bias_dtype,
                            const void* residual, int m, int n, int k, int lda, int ldw, int ldo, float* scratch,
                            long long scratch_floats, int* counters, int n_counters, int* status, int sm_count,
                            int swap, int bn, int splits, int act, const GemmFusion* fusion, cudaStream_t stream);

// x [m][k] (row stride lda), w [n][k] (ldw): bf16.  out, residual [m][n] (ldo), bf16 or fp32 (out_dtype).
// scratch/counters/status: device buffers of the caller; counters must be zero on entry and are zero on return.
FR_EXPORT int gemm_tc(const void* x, const void* w, void* out, int out_dtype, const void* bias, int bias_dtype,
                      const void* residual, int m, int n, int k, int lda, int ldw, int ldo, float* scratch,
                      long long scratch_floats, int* counters, int n_counters, int* status, int sm_count, int swap,
                      int bn, int splits, cudaStream_t stream) {
    return gemm_tc_fused(x, w, out, out_dtype, bias, bias_dtype, residual, m, n, k, lda, ldw, ldo, scratch,
                         scratch_floats, counters, n_counters, status, sm_count, swap, bn, splits, 0, nullptr, stream);
}

// The same with an activation in the epilogue.  act = 1: the rows of w are (gate, up) pairs, n is even, and
// out [m][n/2] (bf16) receives silu(gate) * up; bias and residual must be null.
FR_EXPORT int gemm_tc_act(const void* x, const void* w, void* out, int out_dtype, const void* bias, int bias_dtype,
                          const void* residual, int m, int n, int k, int lda, int ldw, int ldo, float* scratch,
                          long long scratch_floats, int* counters, int n_counters, int* status, int sm_count, int swap,
                          int bn, int splits, int act, cudaStream_t stream) {
    return gemm_tc_fused(x, w, out, out_dtype, bias, bias_dtype, residual, m, n, k, lda, ldw, ldo, scratch,
                         scratch_floats, counters, n_counters, status, sm_count, swap, bn, splits, act, nullptr, stream);
}

// The same with work fused at either end (gemm_tc_fusion.h); fusion may be null.  What a fused part needs of the
// shape is checked here, and refused with the reason: the caller then runs the separate kernels.
FR_EXPORT int gemm_tc_fused(const void* x, const void* w, void* out, int out_dtype, const void* bias, int bias_dtype,
                            const void* residual, int m, int n, int k, int lda, int ldw, int ldo, float* scratch,
                            long long scratch_floats, int* counters, int n_counters, int* status, int sm_count,
                            int swap, int bn, int splits, int act, const GemmFusion* fusion, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return FR_OK;
    if (act != 0 && act != 1) FR_REFUSE("gemm_tc: unknown activation %d", act);
    if (act && (n % 2 || bias != nullptr || residual != nullptr || out_dtype != FR_BF16))
        FR_REFUSE("gemm_tc: the gated epilogue needs an even n, bf16 output, no bias and no residual");
    if (k <= 0 || k % 8 || lda % 8 || ldw % 8)
        FR_REFUSE("gemm_tc: k = %d and the row strides (%d, %d) must be multiples of 8 (16-byte rows for TMA)", k, lda, ldw);
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) FR_REFUSE("gemm_tc: operands must be 16-byte aligned");
    if (status == nullptr) FR_REFUSE("gemm_tc: a status word is needed");
    long long plan[5];
    const bool splits_free = splits < 0;
    gemm_tc_plan(m, n, k, sm_count, swap, bn, splits, plan);
    swap = (int)plan[0]; bn = (int)plan[1]; splits = (int)plan[2];
    const bool narrow_pair = pair_shape(m, n, swap, sm_count) && splits == 1 && bn >= 64 && bn < 128 && bn % 16 == 0;
    if (bn != 16 && bn != 32 && bn != 64 && !(bn >= 128 && bn <= 256 && bn % 16 == 0) && !narrow_pair) FR_REFUSE("gemm_tc: tile width %d", bn);
    // Few rows stream the weights once, and an SM draws only so much (about 45 GB/s on a B200): the product is as fast as
    // its share of busy SMs.  Several waves of whole tiles can leave most SMs idle in the last one (the head's 1,188 tiles
    // on 148 SMs: a ninth wave of four); with FRIDAY_GEMM_EVEN_RUNS=1 the k blocks of all tiles are then laid end to end
    // and cut into equal runs, one per SM, whatever tiles a run touches (its first and last tile are partial tiles that
    // the last CTA to arrive sums).
    bool even_runs = false;
    if (splits_free && swap && use_even_runs()) {
        const long long tiles_now = (long long)((n + TILE_P - 1) / TILE_P) * ((m + bn - 1) / bn);
        const long long items = tiles_now * splits, waves = (items + sm_count - 1) / sm_count;
        const long long kb_all = tiles_now * ((k + TILE_K - 1) / TILE_K);
        if (waves > 1 && items * 10 < waves * sm_count * 9 && kb_all >= 4LL * sm_count && 2LL * sm_count * TILE_P * bn <= scratch_floats &&
            tiles_now <= n_counters) {
            even_runs = true;
            splits = 1;
        }
    }
    if (plan[3] > scratch_floats || plan[4] > n_counters)
        FR_REFUSE("gemm_tc: split-k needs %lld scratch floats and %lld counters, given %lld and %d", plan[3], plan[4],
                  scratch_floats, n_counters);
    GemmParams p;
    p.f = GemmFusion{};
    if (fusion != nullptr) {
        p.f = *fusion;
        const GemmFusion& f = p.f;
        const bool rope = f.row_pos != nullptr || f.row_seq != nullptr || f.denom != nullptr || f.k_pool != nullptr;
        if (f.in_ssq != nullptr && (f.in_parts <= 0 || !(f.in_width > 0.f) || (swap && bn > TILE_P)))
            FR_REFUSE("gemm_tc: a deferred norm of the input needs its partial sums, the width, and tiles of at most %d rows", TILE_P);
        if (rope || (f.norm_out != nullptr && swap)) {
            // both work on the staged tile of the swapped orientation: whole tiles of 128 columns, rows of 16-byte pieces
            if (!swap || act || out_dtype != FR_BF16 || bn > (rope ? 64 : 128) || n % TILE_P || ldo % 8 ||
                (((uintptr_t)out | (uintptr_t)residual | (uintptr_t)f.norm_out) & 15))
                FR_REFUSE("gemm_tc: a fused norm or rotation needs few rows (swapped tiles up to 128 wide, 64 with a rotation), "
                          "bf16 output without activation, n a multiple of %d and 16-byte aligned rows", TILE_P);
        }
        if (f.norm_out != nullptr && !swap) {
            // rows on the M side: every thread finishes whole groups of 16 columns of its row
            if (act || out_dtype != FR_BF16 || n % 16 || ldo % 8 || 
                (((uintptr_t)out | (uintptr_t)residual | (uintptr_t)f.norm_out) & 15))
                FR_REFUSE("gemm_tc: a fused norm needs bf16 output without activation, n a multiple of 16 and 16-byte "
                          "aligned rows");
        }
        if (f.norm_out != nullptr && (f.norm_w == nullptr || f.out_ssq == nullptr))
            FR_REFUSE("gemm_tc: a fused norm needs its weight and a buffer for the sums of squares");
        if (rope) {
            if (f.row_pos == nullptr || f.row_seq == nullptr) FR_REFUSE("gemm_tc: rotation and cache write need row_seq and row_pos");
            if (f.hd <= 0 || TILE_P % f.hd || f.hd % 8 || (long long)(f.nq + 2 * f.nkv) * f.hd != n)
                FR_REFUSE("gemm_tc: fused rotation needs a head size that divides %d and n = (q + 2 kv heads) * head size", TILE_P);
            if (f.denom != nullptr && (f.rot <= 0 || f.rot > f.hd || f.rot % 16))
                FR_REFUSE("gemm_tc: fused rotation needs a rotary size (%d) that is a multiple of 16, at most the head size %d", f.rot, f.hd);
            if (bn > 64 || f.norm_out != nullptr || residual != nullptr)
                FR_REFUSE("gemm_tc: fused rotation needs at most 64 rows and goes without residual or fused norm");
            if (f.k_pool != nullptr && (f.v_pool == nullptr || f.table == nullptr || f.page <= 0 ||
                                        (((uintptr_t)f.k_pool | (uintptr_t)f.v_pool) & 15)))
                FR_REFUSE("gemm_tc: cache write asked for without a whole cache");
        }
    }
    p.out = out; p.bias = bias; p.residual = residual; p.ws = scratch; p.counters = counters; p.status = status;
    p.p_rows = swap ? n : m; p.q_rows = swap ? m : n; p.ldo = ldo; p.out_dtype = out_dtype; p.bias_dtype = bias_dtype;
    p.swapped = swap;
    p.bn = bn;
    p.act = act;
    p.tiles_p = (p.p_rows + TILE_P - 1) / TILE_P; p.tiles_q = (p.q_rows + bn - 1) / bn;
    p.splits = splits; p.kb_total = (k + TILE_K - 1) / TILE_K; p.kb_per = (p.kb_total + splits - 1) / splits;
    // A last wave that would leave most SMs idle is spread over all of them instead (stream-k), if the scratch
    // buffer holds two partial tiles per CTA.
    const int tiles = p.tiles_p * p.tiles_q;
    p.dp_tiles = tiles; p.sk_tiles = 0; p.sk_units = 1;
    int grid = tiles * splits < sm_count ? tiles * splits : sm_count;
    if (even_runs) {
        p.dp_tiles = 0;
        p.sk_tiles = tiles;
        p.sk_units = (int)(((long long)tiles * p.kb_total + sm_count - 1) / sm_count);
        grid = (int)(((long long)tiles * p.kb_total + p.sk_units - 1) / p.sk_units);
    } else if (!swap && splits == 1 && tiles > sm_count && use_stream_k()) {
        const int rem = tiles % sm_count;
        if (rem != 0 && rem * 100 < sm_count * 85 && p.kb_total >= 4 && 2LL * sm_count * TILE_P * bn <= scratch_floats &&
            tiles <= n_counters) {
            p.sk_tiles = rem;
            p.dp_tiles = tiles - rem;
            p.sk_units = (rem * p.kb_total + sm_count - 1) / sm_count;
            grid = sm_count;
        }
    }
    if (pair_shape(m, n, swap, sm_count) && splits == 1 && (bn >= 128 || narrow_pair) && p.sk_tiles == 0) {
        // 256 x bn tiles on pairs of SMs; each CTA loads half of a tile's weight rows
        p.tiles_p = (m + 2 * TILE_P - 1) / (2 * TILE_P);
        const int pair_tiles = p.tiles_p * p.tiles_q;
        p.dp_tiles = pair_tiles;
        CUtensorMap mp, mq;
        int rc = make_map(&mp, x, m, k, lda, TILE_P);
        if (rc) return rc;
        rc = make_map(&mq, w, n, k, ldw, bn / 2);
        if (rc) return rc;
        static std::atomic<unsigned long long> configured{0};
        unsigned long long bit = 0;
        rc = current_device_bit(&bit);
        if (rc) return rc;
        if (!(configured.load(std::memory_order_acquire) & bit)) {
            FR_CUDA(cudaFuncSetAttribute(gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES));
            configured.fetch_or(bit, std::memory_order_release);
        }
        const int pairs = pair_tiles < sm_count / 2 ? pair_tiles : sm_count / 2;
        FR_CUDA(fr_launch_cluster(gemm_tc_pair_kernel, dim3(2 * pairs), dim3(THREADS), PAIR_SMEM_BYTES, stream, 2u, mp, mq, p));
        FR_CHECK_LAUNCH("gemm_tc (pairs)");
        return FR_OK;
    }
    // (up to four rows are one group of a 16-wide tile: one CTA would finish them while the others only wait for it; the
    // last CTA to arrive does it sooner: 354.6 against 352.2 tok/s at batch 1)
    p.shared_finish = swap && splits > 1 && bn <= 128 && m > 4 && grid == tiles * splits && grid <= sm_count && n % TILE_P == 0 &&
                      2 * tiles <= n_counters && use_shared_finish();
    CUtensorMap mp, mq;
    int rc = swap ? make_map(&mp, w, n, k, ldw, TILE_P) : make_map(&mp, x, m, k, lda, TILE_P);
    if (rc) return rc;
    rc = swap ? make_map(&mq, x, m, k, lda, bn) : make_map(&mq, w, n, k, ldw, bn);
    if (rc) return rc;
    switch (bn) {
        case 16: return launch<16, 10>(mp, mq, p, grid, stream);
        case 32: return launch<32, 9>(mp, mq, p, grid, stream);
        case 64: return launch<64, 8>(mp, mq, p, grid, stream);
        case 128: return launch<128, 6>(mp, mq, p, grid, stream);
        default: return launch<256, 4>(mp, mq, p, grid, stream);       // any width from 144 to 256
    }
}

// ------------------------------------------------------------------ the entry point that allocates nothing
#include "gemm_tc_noalloc.h"

namespace {

// Tile counters first (they must start at zero), partial tiles after them.  In host code this name is only
// a stand-in for the symbol: the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char noalloc_area[GEMM_TC_NOALLOC_BYTES];

struct NoAllocDevice {
    bool ready = false;
    unsigned char* base = nullptr;     // device address of noalloc_area on this device
    int sm_count = 0;
};
NoAllocDevice noalloc_devices[64];
std::mutex noalloc_mutex;          // the first calls of two host threads on one device must not both fill the entry

template <int BN, int STAGES>
cudaError_t allow_smem() {
    return cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                smem_bytes<BN, STAGES>());
}

// Once per device, with that device current.
int noalloc_setup(int device) {
    NoAllocDevice& d = noalloc_devices[device];
    void* ptr = nullptr;
    FR_CUDA(cudaGetSymbolAddress(&ptr, noalloc_area));
    FR_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device));
    FR_CUDA((allow_smem<16, 10>()));
    FR_CUDA((allow_smem<32, 9>()));
    FR_CUDA((allow_smem<64, 8>()));
    FR_CUDA((allow_smem<128, 6>()));
    FR_CUDA((allow_smem<256, 4>()));
    d.base = (unsigned char*)ptr;
    d.ready = true;
    return FR_OK;
}

}  // namespace

FR_EXPORT int gemm_tc_noalloc(const void* x, const void* w, void* out, int out_dtype, const void* bias,
                              int bias_dtype, const void* residual, int m, int n, int k, int lda, int ldw, int ldo,
                              int* status, cudaStream_t stream) {
    int device = 0;
    FR_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= 64) FR_REFUSE("gemm_tc_noalloc: device %d is outside the table of 64", device);
    {
        std::lock_guard<std::mutex> lock(noalloc_mutex);
        if (!noalloc_devices[device].ready) {
            const int rc = noalloc_setup(device);
            if (rc) return rc;
        }
    }
    const NoAllocDevice& d = noalloc_devices[device];
    if (m <= 0 || n <= 0) return FR_OK;
    long long plan[5];
    gemm_tc_plan(m, n, k > 0 ? k : 1, d.sm_count, -1, -1, -1, plan);
    if (plan[3] > GEMM_TC_NOALLOC_SCRATCH_FLOATS || plan[4] > GEMM_TC_NOALLOC_COUNTERS)
        FR_REFUSE("gemm_tc_noalloc: a product of %d x %d x %d splits k %lld ways over %lld tiles and needs %lld scratch "
                  "floats; the built-in area holds %d floats and %d tiles. Use gemm_tc() with a buffer of your own.",
                  m, n, k, plan[2], plan[4], plan[3], GEMM_TC_NOALLOC_SCRATCH_FLOATS, GEMM_TC_NOALLOC_COUNTERS);
    int* counters = (int*)d.base;
    float* scratch = (float*)(d.base + GEMM_TC_NOALLOC_COUNTERS * 4);
    // The area keeps what the last call left; counters must start at zero whatever happened before.
    FR_CUDA(cudaMemsetAsync(counters, 0, GEMM_TC_NOALLOC_COUNTERS * 4, stream));
    return gemm_tc(x, w, out, out_dtype, bias, bias_dtype, residual, m, n, k, lda, ldw, ldo, scratch,
                   GEMM_TC_NOALLOC_SCRATCH_FLOATS, counters, GEMM_TC_NOALLOC_COUNTERS, status, d.sm_count, (int)plan[0],
                   (int)plan[1], (int)plan[2], stream);
}
