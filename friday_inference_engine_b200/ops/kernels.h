// The kernel libraries (one shared library per file of csrc/) and their C entry points.
//
// A library is opened when it is first needed, from the folder that holds this library
// (or $FRIDAY_BUILD_DIR).  If it is not there, the builder hook is asked for it (the
// Python package compiles the family with nvcc at that moment); without a hook, or if
// the library still cannot be opened, the call fails with a KernelError that says how to
// build.  Nothing falls back to another path.
#pragma once
#include <cuda_runtime.h>

#include <string>

#include "csrc/gemm_tc_fusion.h"

namespace friday {
namespace kernels {

typedef const char* (*last_error_fn)();

struct Rowwise {
    last_error_fn last_error;
    int (*embedding)(const int*, const void*, void*, int, int, int, int, cudaStream_t);
    int (*gather_rows)(const int*, const void*, void*, int, int, int, cudaStream_t);
    int (*rmsnorm)(const void*, const void*, int, void*, int, int, float, int, cudaStream_t);
    int (*swiglu)(const void*, void*, int, int, int, cudaStream_t);
    int (*rope_kv_write)(void*, const int*, const int*, const float*, int, int, int, int, void*, void*, const int*, int, int,
                         int, int, int, cudaStream_t);
    int (*advance)(int*, const int*, int*, int*, const int*, int*, int, cudaStream_t);
    int (*scale_rows)(void*, long long, float, int, cudaStream_t);
    int (*finish_logits)(float*, int, int, int, const void*, int, float, float, cudaStream_t);
    int (*random_normal)(void*, long long, int, unsigned long long, float, float, cudaStream_t);
};
struct GemmSimt {
    last_error_fn last_error;
    int (*gemm)(const void*, int, const void*, int, void*, int, const void*, int, const void*, int, int, int, int, int, int,
                cudaStream_t);
};
struct GemmTc {
    last_error_fn last_error;
    int (*fused)(const void*, const void*, void*, int, const void*, int, const void*, int, int, int, int, int, int, float*,
                 long long, int*, int, int*, int, int, int, int, int, const GemmFusion*, cudaStream_t);
    int (*plan)(int, int, int, int, int, int, int, long long*);
};
struct AttentionSimt {
    last_error_fn last_error;
    int (*run)(const void*, int, void*, const void*, const void*, const int*, int, int, const int*, const int*, int, int, int,
               int, int, float, int, float*, int, cudaStream_t);
};
struct AttentionMma {
    last_error_fn last_error;
    int (*run)(const void*, int, void*, const void*, const void*, int, const int*, int, int, const int*, const int*,
               const int*, const int*, int, int, int, int, int, int, int, float, int, int, float*, int*, int, int*,
               cudaStream_t);
    int (*clusters_at_once)(int, int);
};
struct AttentionTc {
    last_error_fn last_error;
    int (*run)(const void*, int, int, void*, const void*, const void*, int, const int*, int, const int*, const int*,
               const int*, const int*, int, int, int, int, int, int, float, int*, cudaStream_t);
};
struct Sampling {
    last_error_fn last_error;
    int (*sample)(const float*, int, int, int, const float*, const int*, const int*, unsigned long long, const int*, int*,
                  cudaStream_t);
};

const Rowwise& rowwise();
const GemmSimt& gemm_simt();
const GemmTc& gemm_tc();
const AttentionSimt& attention_simt();
const AttentionMma& attention_mma();
const AttentionTc& attention_tc();
const Sampling& sampling();

// Called with a family's name when its library is missing; returns 0 when it has built it.
typedef int (*builder_fn)(const char* family);
void set_builder(builder_fn f);
std::string library_dir();
std::string loaded_libraries();     // paths, one per line

}  // namespace kernels
}  // namespace friday
