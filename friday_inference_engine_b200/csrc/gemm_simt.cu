// out[m][n] = sum_k a[m][k] * w[n][k]  (+ bias[n]) (+ residual[m][n])
//
// CUDA-core matrix product with fp32 multiply-adds in the order of k: the true
// 32-bit path of the model (no tensor cores, no reduced-precision mode), and the
// fallback of the bf16 path for sizes that the tensor-core kernel refuses.  Both
// operands are row-major with k innermost, which is how activations [rows][k] and
// projection weights [out][in] are stored, so nothing is transposed.  Any m, n, k.
//
// The reference's counterpart is its int8 tensor-core GEMM with the same epilogue
// (bias, then residual, in place allowed): prefill_kernels.cu:156-171, 173-327.
#include "common.cuh"

FR_EXPORT const char* gemm_simt_last_error() { return fr_error_text; }

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;   // 256 threads, 4x4 outputs each

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ a, const TW* __restrict__ w, TO* out, FrVec bias, const TO* residual, int m,
                 int n, int k, int lda, int ldw, int ldo) {
    __shared__ float as[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;     // tx: 4 columns, ty: 4 rows
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < k; k0 += BK) {
        // 64 x 16 elements per operand, 4 per thread; consecutive threads read consecutive k.
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int idx = tid + r * 256;
            const int row = idx / BK, kk = idx % BK;
            const int gk = k0 + kk;
            float va = 0.f, vw = 0.f;
            if (gk < k) {
                if (m0 + row < m) va = fr_load(a + (size_t)(m0 + row) * lda + gk);
                if (n0 + row < n) vw = fr_load(w + (size_t)(n0 + row) * ldw + gk);
            }
            as[kk][row] = va;
            ws[kk][row] = vw;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float ra[TM], rw[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) ra[i] = as[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) rw[j] = ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ra[i], rw[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= m) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn >= n) continue;
            float v = acc[i][j];
            if (bias.p != nullptr) v += bias.at(gn);
            if (residual != nullptr) v += fr_load(residual + (size_t)gm * ldo + gn);
            fr_store(out + (size_t)gm * ldo + gn, v);
        }
    }
}

template <typename TA, typename TW, typename TO>
int launch(const void* a, const void* w, void* out, FrVec bias, const void* residual, int m, int n, int k, int lda,
           int ldw, int ldo, cudaStream_t stream) {
    dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM);
    gemm_simt_kernel<TA, TW, TO><<<grid, 256, 0, stream>>>((const TA*)a, (const TW*)w, (TO*)out, bias,
                                                          (const TO*)residual, m, n, k, lda, ldw, ldo);
    FR_CHECK_LAUNCH("gemm_simt");
    return FR_OK;
}

}  // namespace

// a: [m][k] (row stride lda), w: [n][k] (row stride ldw), out and residual: [m][n]
// (row stride ldo; residual may be `out` itself).  bias may be null; its dtype is
// given apart from the others because a bias stored in 32-bit stays so.
FR_EXPORT int gemm_simt(const void* a, int a_dtype, const void* w, int w_dtype, void* out, int out_dtype,
                        const void* bias, int bias_dtype, const void* residual, int m, int n, int k, int lda,
                        int ldw, int ldo, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return FR_OK;
    if (k <= 0) FR_REFUSE("gemm_simt: k = %d", k);
    FrVec bv{bias, bias_dtype};
    typedef __nv_bfloat16 bf16;
    const int key = a_dtype * 4 + w_dtype * 2 + out_dtype;
    switch (key) {
        case 0: return launch<float, float, float>(a, w, out, bv, residual, m, n, k, lda, ldw, ldo, stream);
        case 4: return launch<bf16, float, float>(a, w, out, bv, residual, m, n, k, lda, ldw, ldo, stream);
        case 5: return launch<bf16, float, bf16>(a, w, out, bv, residual, m, n, k, lda, ldw, ldo, stream);
        case 6: return launch<bf16, bf16, float>(a, w, out, bv, residual, m, n, k, lda, ldw, ldo, stream);
        case 7: return launch<bf16, bf16, bf16>(a, w, out, bv, residual, m, n, k, lda, ldw, ldo, stream);
        default: FR_REFUSE("gemm_simt: no kernel for dtypes a=%d w=%d out=%d", a_dtype, w_dtype, out_dtype);
    }
}
