// Device-side building blocks of the tensor-core kernels: mbarrier, TMA, tcgen05 and descriptor helpers,
// bounded waits, and the epilogue that turns 16 accumulator columns into stored outputs.  Shared by the matrix
// product (gemm_tc.cu, gemm_tc_pair.cuh) and the attention kernels that use tcgen05 and TMA.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace tc {

constexpr int TILE_P = 128;          // rows of P per tile = M of the instruction
constexpr int TILE_K = 64;           // bf16 elements per stage along k = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int P_BYTES = TILE_P * TILE_K * 2;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // a wait gives up after two seconds

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait; false (and a code in *status) if the barrier did not complete in time.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
    if (mbar_try(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try(bar, parity)) return true;
        if ((it & 63u) == 0 && global_ns() - t0 > WAIT_LIMIT_NS) break;
    }
    atomicCAS(status, 0, code);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}
// One lane of a converged warp (the compiler sees that exactly one lane runs what follows, and may keep the
// operands of tcgen05 instructions in uniform registers instead of converting them for every instruction).
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n.reg .pred p;\n"
        "elect.sync _|p, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows of 128 bytes,
// groups of 8 rows 1024 bytes apart.  Bits: [0,14) address >> 4; [16,30) leading byte
// offset >> 4 (unused with this swizzle); [32,46) stride byte offset >> 4; [46,48) = 1
// (descriptor version of sm_100); [61,64) = 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor of kind::f16: fp32 accumulate (bit 4), bf16 A (bit 7) and B (bit 10), both
// K-major (bits 15, 16 clear), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

template <typename P>
__device__ __forceinline__ float bias_at(const P& p, int i) {
    return p.bias_dtype == FR_F32 ? ((const float*)p.bias)[i] : __bfloat162float(((const __nv_bfloat16*)p.bias)[i]);
}

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }

// Gated epilogue: rows 2f and 2f+1 of the weight are gate f and up f.  Must be called by whole warps.
template <typename P>
__device__ __forceinline__ void finish16_gated(const P& p, int gi, int gj0, float (&v)[16]) {
    if (!p.swapped) {
        // the pair sits in one thread: columns gj0 + 2j, gj0 + 2j + 1 -> out[gi][gj0/2 + j]
        if (gi >= p.p_rows) return;
        float r[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] = silu_mul(v[2 * j], v[2 * j + 1]);
        const int oj0 = gj0 >> 1, o_cols = p.q_rows >> 1;
        __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)gi * p.ldo + oj0;
        if (oj0 + 8 <= o_cols && (p.ldo % 8 == 0) && (((uintptr_t)p.out & 15) == 0)) {
            uint4 pk;
            __nv_bfloat162* ph = (__nv_bfloat162*)&pk;
#pragma unroll
            for (int j = 0; j < 4; ++j) ph[j] = __floats2bfloat162_rn(r[2 * j], r[2 * j + 1]);
            *(uint4*)o = pk;
        } else {
            for (int j = 0; j < 8 && oj0 + j < o_cols; ++j) o[j] = __float2bfloat16_rn(r[j]);
        }
    } else {
        // the pair sits in neighbouring lanes (TMEM lanes are weight rows): out[gj][gi/2]
        float up[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) up[j] = __shfl_xor_sync(0xffffffffu, v[j], 1);
        if ((gi & 1) || gi >= p.p_rows) return;
        for (int j = 0; j < 16 && gj0 + j < p.q_rows; ++j)
            ((__nv_bfloat16*)p.out)[(size_t)(gj0 + j) * p.ldo + (gi >> 1)] = __float2bfloat16_rn(silu_mul(v[j], up[j]));
    }
}

// Bias, residual, rounding and store of 16 consecutive q-columns of P-row gi.
template <typename P>
__device__ __forceinline__ void finish16(const P& p, int gi, int gj0, float (&v)[16]) {
    if (p.act) return finish16_gated(p, gi, gj0, v);
    if (gi >= p.p_rows) return;
    if (!p.swapped) {
        // out[gi][gj0 .. gj0+15]
        const size_t base = (size_t)gi * p.ldo + gj0;
        const bool whole = gj0 + 16 <= p.q_rows;
        if (p.out_dtype == FR_BF16) {
            __nv_bfloat16* o = (__nv_bfloat16*)p.out + base;
            const __nv_bfloat16* r = p.residual ? (const __nv_bfloat16*)p.residual + base : nullptr;
            if (whole && (p.ldo % 8 == 0) && (((uintptr_t)p.out & 15) == 0) &&
                (r == nullptr || ((uintptr_t)p.residual & 15) == 0)) {
                if (p.bias)
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] += bias_at(p, gj0 + j);
                if (r) {
                    uint4 rr[2] = {((const uint4*)r)[0], ((const uint4*)r)[1]};
                    const __nv_bfloat16* rb = (const __nv_bfloat16*)rr;
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] += __bfloat162float(rb[j]);
                }
                uint4 pk[2];
                __nv_bfloat162* ph = (__nv_bfloat162*)pk;
#pragma unroll
                for (int j = 0; j < 8; ++j) ph[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                ((uint4*)o)[0] = pk[0];
                ((uint4*)o)[1] = pk[1];
            } else {
                for (int j = 0; j < 16 && gj0 + j < p.q_rows; ++j) {
                    float x = v[j];
                    if (p.bias) x += bias_at(p, gj0 + j);
                    if (r) x += __bfloat162float(r[j]);
                    o[j] = __float2bfloat16_rn(x);
                }
            }
        } else {
            float* o = (float*)p.out + base;
            const float* r = p.residual ? (const float*)p.residual + base : nullptr;
            if (whole && (p.ldo % 4 == 0) && (((uintptr_t)p.out & 15) == 0) && r == nullptr) {
                if (p.bias)
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] += bias_at(p, gj0 + j);
#pragma unroll
                for (int j = 0; j < 4; ++j) ((float4*)o)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            } else {
                for (int j = 0; j < 16 && gj0 + j < p.q_rows; ++j) {
                    float x = v[j];
                    if (p.bias) x += bias_at(p, gj0 + j);
                    if (r) x += r[j];
                    o[j] = x;
                }
            }
        }
    } else {
        // transposed: out[gj][gi]; bias goes with gi.  The residual may be `out` itself, so the compiler must keep
        // every load before the store that follows it: all loads are issued first, then all stores, or the 16
        // columns would cost 16 round trips to memory one after the other.
        const float b = p.bias ? bias_at(p, gi) : 0.f;
        const int n = min(16, p.q_rows - gj0);
        float r[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            r[j] = 0.f;
            if (p.residual != nullptr && j < n) {
                const size_t at = (size_t)(gj0 + j) * p.ldo + gi;
                if (p.out_dtype == FR_BF16) {
                    const unsigned short raw = __ldcg((const unsigned short*)p.residual + at);
                    r[j] = __uint_as_float((uint32_t)raw << 16);
                } else {
                    r[j] = __ldcg((const float*)p.residual + at);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            if (j < n) {
                const size_t at = (size_t)(gj0 + j) * p.ldo + gi;
                const float x = v[j] + b + r[j];
                if (p.out_dtype == FR_BF16) ((__nv_bfloat16*)p.out)[at] = __float2bfloat16_rn(x);
                else ((float*)p.out)[at] = x;
            }
        }
    }
}


}  // namespace tc
