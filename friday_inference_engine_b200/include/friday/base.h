// Errors, storage types and the tensor descriptor that every part of the library shares.
//
// A Tensor names device memory; it owns nothing.  Memory belongs to whoever made it:
// the weights' store, the cache's pools, or an Arena that hands out the rows of one
// pass and takes them all back at once.  The reference does the same with raw pointers
// into a few long-lived buffers (transformer.h:139-176).
#pragma once
#include <stdint.h>

#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace friday {

// ---- errors: one class per kind of mistake, so that callers (and the bindings) can tell them apart
enum class ErrorKind : int { Other = 0, Config = 1, Weights = 2, Step = 3, Cache = 4, CacheFull = 5, Generation = 6,
                             Kernel = 7, Build = 8 };

struct Error : std::runtime_error {
    ErrorKind kind;
    Error(ErrorKind k, const std::string& what) : std::runtime_error(what), kind(k) {}
};
struct ConfigError : Error { explicit ConfigError(const std::string& w) : Error(ErrorKind::Config, w) {} };
struct StepError : Error { explicit StepError(const std::string& w) : Error(ErrorKind::Step, w) {} };
struct CacheError : Error {
    explicit CacheError(const std::string& w, ErrorKind k = ErrorKind::Cache) : Error(k, w) {}
};
struct CacheFull : CacheError { explicit CacheFull(const std::string& w) : CacheError(w, ErrorKind::CacheFull) {} };
struct GenerationError : Error { explicit GenerationError(const std::string& w) : Error(ErrorKind::Generation, w) {} };
struct KernelError : Error { explicit KernelError(const std::string& w) : Error(ErrorKind::Kernel, w) {} };
struct BuildError : Error { explicit BuildError(const std::string& w) : Error(ErrorKind::Build, w) {} };

struct ShapeMismatch {
    std::string name;
    std::vector<int64_t> got, want;
};
// One error for everything that is wrong between a model and a weight source.
struct WeightsError : Error {
    std::vector<std::string> missing, unexpected;
    std::vector<ShapeMismatch> wrong_shape;
    explicit WeightsError(const std::string& w) : Error(ErrorKind::Weights, w) {}
};

std::string format(const char* fmt, ...) __attribute__((format(printf, 1, 2)));

// ---- storage
enum class DType : int { F32 = 0, BF16 = 1, I32 = 2 };      // F32 and BF16 are the kernels' dtype codes

inline size_t dtype_size(DType d) { return d == DType::BF16 ? 2 : 4; }
const char* dtype_name(DType d);
DType parse_dtype(const std::string& name);                  // "bfloat16" | "bf16" | "float32" | "fp32" | "f32"

struct Tensor {
    void* data = nullptr;
    DType dtype = DType::F32;
    int ndim = 0;
    int64_t shape[4] = {0, 0, 0, 0};
    int64_t ld = 0;          // elements from one row to the next (rows = all dimensions but the last)

    bool defined() const { return data != nullptr; }
    int64_t cols() const { return ndim ? shape[ndim - 1] : 1; }
    int64_t rows() const {
        int64_t r = 1;
        for (int i = 0; i + 1 < ndim; ++i) r *= shape[i];
        return r;
    }
    int64_t numel() const { return rows() * cols(); }
    size_t bytes() const { return (size_t)numel() * dtype_size(dtype); }
    bool contiguous() const { return ld == cols(); }
    std::vector<int64_t> dims() const { return std::vector<int64_t>(shape, shape + ndim); }

    static Tensor make(void* p, DType dt, std::initializer_list<int64_t> dims) {
        Tensor t;
        t.data = p;
        t.dtype = dt;
        for (int64_t d : dims) t.shape[t.ndim++] = d;
        t.ld = t.cols();
        return t;
    }
    static Tensor make(void* p, DType dt, const std::vector<int64_t>& dims) {
        Tensor t;
        t.data = p;
        t.dtype = dt;
        for (int64_t d : dims) t.shape[t.ndim++] = d;
        t.ld = t.cols();
        return t;
    }
    // rows [r0, r0 + n) of a 2-d tensor
    Tensor row_slice(int64_t r0, int64_t n) const {
        Tensor t = *this;
        t.data = (char*)data + (size_t)r0 * ld * dtype_size(dtype);
        t.shape[0] = n;
        return t;
    }
    // item i of the first dimension of a contiguous tensor of 2 or more dimensions
    Tensor index0(int64_t i) const {
        Tensor t;
        t.dtype = dtype;
        t.ndim = ndim - 1;
        int64_t inner = 1;
        for (int k = 1; k < ndim; ++k) {
            t.shape[k - 1] = shape[k];
            inner *= shape[k];
        }
        t.ld = t.cols();
        t.data = (char*)data + (size_t)i * inner * dtype_size(dtype);
        return t;
    }
};

}  // namespace friday
