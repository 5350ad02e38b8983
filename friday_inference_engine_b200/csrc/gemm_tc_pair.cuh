// The matrix product of many rows on pairs of SMs: two CTAs of a cluster share one 256 x bn tile
// (tcgen05.mma.cta_group::2).  Each CTA loads its own 128 rows of the activations and HALF of the tile's weight
// rows; the instruction, issued by the pair's first CTA, reads both halves.  Per 128 x bn of output a CTA then
// moves 16 KB + bn * 64 bytes per k block into shared memory instead of 16 KB + bn * 128: the product of a
// prompt is bound by exactly that traffic and by the power it costs.
//
// Included by gemm_tc.cu (after its parameter structs and epilogue helpers); rows on the M side only, every tile
// computed whole (no split of k).  The protocol between the two CTAs:
//   * stage s of the ring is filled by both CTAs' TMA warps; all four loads signal the FIRST CTA's full[s], which
//     expects the bytes of both;
//   * the first CTA's MMA thread waits for full[s], issues the instructions, and commits to empty[s] of BOTH CTAs
//     (a multicast commit), after a tile's last k block to acc_full[a] of both;
//   * both CTAs' epilogue warps read their own 128 lanes of the accumulator and arrive on the FIRST CTA's
//     acc_empty[a] (eight arrivals).
// Every wait is bounded as in gemm_tc.cu.  Neither CTA leaves before the other (a cluster barrier before tensor
// memory is freed): a CTA's shared memory and barriers are written from outside until the pair is done.
#pragma once

namespace {

constexpr int PAIR_BN = 256;                          // widest tile; p.bn may be any multiple of 16 up to it
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_Q_BYTES = (PAIR_BN / 2) * TILE_K * 2;
constexpr int PAIR_STAGE_BYTES = P_BYTES + PAIR_Q_BYTES;
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + (2 * PAIR_STAGES + 4) * 8 + 64 + PAIR_BN * 4;

__device__ __forceinline__ uint32_t cluster_addr(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
// `bar` is a shared::cluster address: the barrier may be the other CTA's.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives, once the instructions issued so far are done, on the barrier at this offset in both CTAs of the pair
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3)
                 : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q, const GemmParams p) {
    constexpr int STAGES = PAIR_STAGES, STAGE_BYTES = PAIR_STAGE_BYTES, BN = PAIR_BN;
    constexpr int TMEM_COLS = 2 * BN;
    const int bn = p.bn, half = bn >> 1;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);
    // bars: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    float* s_gw = (float*)((uint8_t*)(bars + 2 * STAGES + 4) + 64);         // [BN] norm weights of the tile's columns
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = fr_cluster_rank();                                 // 0: the CTA that issues the instructions
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t accf0 = smem_u32(bars + 2 * STAGES), acce0 = smem_u32(bars + 2 * STAGES + 2);
    const uint32_t first_full0 = cluster_addr(full0, 0), first_acce0 = cluster_addr(acce0, 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(accf0 + 8 * a, 1);
            mbar_init(acce0 + 8 * a, 8);                   // the epilogue warps of both CTAs
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    fr_cluster_sync();                                     // the other CTA's barriers are ready before anything reaches them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) fr_pdl_launch();

    if (warp == 0) {
        if (elect_one()) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_p) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
            struct Walk {                                  // the k blocks this pair will load, in order
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
            const uint32_t stage_tx = 2u * (P_BYTES + (uint32_t)half * TILE_K * 2);      // both CTAs' bytes of a stage
            Walk head(p, pair, pairs);
            Walk ahead(p, pair, pairs);
            int early = 0;
            for (; early < STAGES && ahead.live; ++early, ahead.step(p)) {
                if (rank == 0) mbar_expect_tx(full0 + 8 * early, stage_tx);
                tma_load_2d_pair(smem_u32(smem + early * STAGE_BYTES) + P_BYTES, &map_q, ahead.kb * TILE_K,
                                 ahead.q_blk * bn + (int)rank * half, first_full0 + 8 * early);
            }
            fr_pdl_wait();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (; head.live && ok; head.step(p)) {
                const uint32_t dst = smem_u32(smem + stage * STAGE_BYTES);
                if (early > 0) {
                    --early;                                 // the weight slice of this stage is already on its way
                } else {
                    if (!(ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, p.status, 1))) break;
                    if (rank == 0) mbar_expect_tx(full0 + 8 * stage, stage_tx);
                    tma_load_2d_pair(dst + P_BYTES, &map_q, head.kb * TILE_K, head.q_blk * bn + (int)rank * half,
                                     first_full0 + 8 * stage);
                }
                tma_load_2d_pair(dst, &map_p, head.kb * TILE_K, (2 * head.p_blk + (int)rank) * TILE_P, first_full0 + 8 * stage);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        if (rank == 0 && elect_one()) {
            fr_pdl_wait();
            const uint32_t idesc = instr_desc(2 * TILE_P, bn);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int it = 0;
            Work work(p, pair, pairs);
            Item item;
            for (; ok && work.next(item); ++it) {
                const int a = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!(ok = mbar_wait(acce0 + 8 * a, acc_phase ^ 1, p.status, 2))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + a * BN;
                for (int kb = item.kb0; kb < item.kb1; ++kb) {
                    if (!(ok = mbar_wait(full0 + 8 * stage, phase, p.status, 3))) break;
                    tc_fence_after();
                    const uint32_t pa = smem_u32(smem + stage * STAGE_BYTES);
                    const uint64_t da = smem_desc(pa), db = smem_desc(pa + P_BYTES);
#pragma unroll
                    for (int k = 0; k < TILE_K / UMMA_K; ++k)
                        tc_mma_pair(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > item.kb0 || k > 0) ? 1u : 0u);
                    tc_commit_pair(empty0 + 8 * stage);   // the stage is free in both CTAs once these products are done
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) tc_commit_pair(accf0 + 8 * a);    // the accumulator is complete, in both CTAs
            }
        }
    } else {
        const int quarter = warp & 3;                      // TMEM lanes this warp may read: 32*quarter ..
        const int i_local = quarter * 32 + lane;
        const int et = threadIdx.x - 64;                   // 0..127 among the epilogue threads
        fr_pdl_wait();
        bool ok = true;
        int it = 0;
        const GemmFusion& f = p.f;
        const bool norm_rows = f.norm_out != nullptr;
        int scale_blk = -1;
        float row_scale = 1.f;
        Work work(p, pair, pairs);
        Item item;
        for (; ok && work.next(item); ++it) {
            const int q_blk = item.tile / p.tiles_p, p_blk = 2 * (item.tile - q_blk * p.tiles_p) + (int)rank;
            const int a = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            const int gi = p_blk * TILE_P + i_local;
            if (f.in_ssq != nullptr && p_blk != scale_blk) {
                // the deferred norm of the input: the factor of this thread's row
                float ss = 0.f;
                if (gi < p.p_rows)
                    for (int t = 0; t < f.in_parts; ++t) ss += __ldcg(f.in_ssq + (size_t)t * p.p_rows + gi);
                row_scale = 1.0f / sqrtf(ss / f.in_width + f.in_eps);
                scale_blk = p_blk;
            }
            float ss_row = 0.f;                            // with a norm begun: this row's sum of squares over the tile
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
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + a * BN;
#pragma unroll 1
            for (int c = 0; c < bn / 16; ++c) {
                uint32_t r[16];
                tc_ld16(taddr + c * 16, r);
                tc_ld_wait();
                float v[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
                if (f.in_ssq != nullptr)
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] *= row_scale;
                const int gj0 = q_blk * bn + c * 16;
                if (norm_rows) finish16_begin_norm(p, s_gw + c * 16, gi, gj0, v, ss_row);
                else finish16(p, gi, gj0, v);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(first_acce0 + 8 * a);     // the accumulator may be overwritten
            if (norm_rows && gi < p.p_rows) f.out_ssq[(size_t)q_blk * p.p_rows + gi] = ss_row;
        }
    }
    tc_fence_before();
    __syncthreads();
    fr_cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

}  // namespace
