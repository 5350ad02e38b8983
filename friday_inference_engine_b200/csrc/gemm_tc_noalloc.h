// gemm_tc_noalloc: the tensor-core matrix product for callers that must not allocate.
//
// This entry point has no counterpart in the reference (onurtamer/friday-inference-engine
// allocates its scratch with cudaMalloc when the model is built: transformer.cpp:270-288).
//
// Who needs it.  The ordinary entry point, gemm_tc(), takes its split-k scratch, tile
// counters and status word from the caller, who normally gets them from an allocator.
// Some hosts have no allocator to ask once they are running: a serving process that
// handed every free byte of device memory to weights and cache at start-up, so that a
// later cudaMalloc fails or forces a trim; a latency-bound loop in which an allocation's
// implicit device synchronisation is not acceptable; a plug-in called from a host
// program that forbids CUDA memory calls in its callbacks; code that has no torch
// allocator in the process at all.  For them the scratch lives inside this library.
//
// What it does.  The same kernel, the same tile choice and split-k as gemm_tc(); partial
// tiles and tile counters go to a file-scope `static __device__` array of
// GEMM_TC_NOALLOC_BYTES bytes (8 MiB + 4 KiB) that every GPU loading the library holds
// until the process exits.  The call allocates nothing: no cudaMalloc, no cudaFree, no
// allocating library routine.
//
// Limits and rules.
//   * A shape whose split-k plan needs more than GEMM_TC_NOALLOC_SCRATCH_FLOATS floats of
//     partial tiles or more than GEMM_TC_NOALLOC_COUNTERS tiles is refused with a message
//     (gemm_tc_last_error()); nothing is launched.  Products with few rows (decoding,
//     up to 64 rows) always fit; wide prompts that would split k may not.
//   * The first call on a device looks the array's address up (cudaGetSymbolAddress, with
//     that device current) and sets the kernels' shared-memory limit, under a lock, so
//     host threads may make their first calls at the same time.  That first call should
//     come before any stream capture.
//   * All calls on a device share the one array, and it keeps what the last call left.
//     The call clears the counters itself; partial tiles are always written before they
//     are read.  Two calls that overlap on the GPU (different streams) race on the array:
//     keep calls on one device in one stream, or order them with events.
//   * x, w, out, bias, residual and status are the caller's, as for gemm_tc(): bf16
//     operands with 16-byte aligned rows, out/residual bf16 or fp32, status a device int
//     that the kernel sets if one of its bounded waits gave up.
#pragma once
#include <cuda_runtime.h>

#define GEMM_TC_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)     /* 8 MiB of partial tiles */
#define GEMM_TC_NOALLOC_COUNTERS 1024                        /* 4 KiB of tile counters */
#define GEMM_TC_NOALLOC_BYTES (GEMM_TC_NOALLOC_SCRATCH_FLOATS * 4 + GEMM_TC_NOALLOC_COUNTERS * 4)

#ifdef __cplusplus
extern "C" {
#endif

// out[m][n] = sum_k x[m][k] * w[n][k] (+ bias[n]) (+ residual[m][n]); returns 0, or a non-zero code with the
// text in gemm_tc_last_error().  Dtype codes: 0 = float32, 1 = bfloat16.  Row strides in elements.
int gemm_tc_noalloc(const void* x, const void* w, void* out, int out_dtype, const void* bias, int bias_dtype,
                    const void* residual, int m, int n, int k, int lda, int ldw, int ldo, int* status,
                    cudaStream_t stream);

#ifdef __cplusplus
}
#endif
