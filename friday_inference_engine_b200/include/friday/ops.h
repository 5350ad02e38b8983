// The operations that parts are made of.  Every one launches this library's own CUDA
// kernels (csrc/) on the Ops object's stream; there is no CPU path, and a kernel library
// that cannot be loaded is an error of the call that needed it.
//
// Memory: results are taken from the Ops object's current Arena, which the caller of a
// pass (the model's run loop) sets and resets; a result lives until the arena that it
// came from is reset.  Weights, cache pools and anything that must outlive a pass are
// allocated by their owners with DeviceBuffer.
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <string>
#include <tuple>
#include <vector>

#include "friday/base.h"
#include "friday/parts.h"

struct GemmFusion;          // csrc/gemm_tc_fusion.h: optional work at the two ends of the tensor-core product

namespace friday {

void cuda_check(cudaError_t e, const char* what);

class DeviceBuffer {
public:
    DeviceBuffer() {}
    explicit DeviceBuffer(size_t bytes, bool zero = false);
    ~DeviceBuffer();
    DeviceBuffer(DeviceBuffer&& o) noexcept : p_(o.p_), n_(o.n_) { o.p_ = nullptr; o.n_ = 0; }
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept;
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    void* get() const { return p_; }
    size_t bytes() const { return n_; }
    template <class T> T* as() const { return (T*)p_; }

private:
    void* p_ = nullptr;
    size_t n_ = 0;
};

// Hands out device memory by bumping an offset; reset() takes everything back.  When a block runs out,
// another is added (earlier results stay where they are); the next reset() joins the blocks into one, after
// which addresses differ from before: generation() counts those events, so that whoever keeps addresses (a
// captured graph) knows when they are stale.
class Arena {
public:
    explicit Arena(cudaStream_t stream, size_t first_block = (size_t)1 << 20) : stream_(stream), first_(first_block) {}
    ~Arena();
    void* alloc(size_t bytes);
    void reset();
    uint64_t generation() const { return generation_; }
    size_t capacity() const;
    bool frozen = false;            // true while a graph is being captured: growing is an error then

private:
    struct BlockMem { void* p; size_t size; };
    std::vector<BlockMem> blocks_;
    size_t offset_ = 0;             // in the last block
    cudaStream_t stream_;
    size_t first_;
    uint64_t generation_ = 0;
};

// Rows on their way from one product to the next.  Plain rows are a tensor.  Deferred rows are rows whose
// RMSNorm the product that made them has begun: `t` holds weight (*) x rounded to bf16, `ssq` [parts, rows]
// each part's share of the rows' sums of squares; the product that takes them finishes the norm by scaling
// its own rows with 1 / sqrt(sum / width + eps).  Anything else asks Ops::materialize, which runs the norm's
// kernel on `source`.
struct Rows {
    Tensor t;
    bool deferred = false;
    Tensor ssq, source, weight;
    float eps = 0;
    Rows() {}
    Rows(const Tensor& x) : t(x) {}
};

struct PartOut {
    Tensor x;                // residual + part(h)
    bool has_normed = false;
    Rows normed;             // `then` of x, if the part produced it
    PartOut() {}
    PartOut(const Tensor& t) : x(t) {}
    PartOut(const Tensor& t, const Rows& n) : x(t), has_normed(true), normed(n) {}
};


class Ops {
public:
    Ops(int device, cudaStream_t stream);
    ~Ops();
    Ops(const Ops&) = delete;

    int device() const { return device_; }
    cudaStream_t stream() const { return stream_; }
    int sm_count() const { return sms_; }
    Arena* arena = nullptr;                                   // where results come from
    Tensor alloc(DType dtype, int64_t rows, int64_t cols);
    float* scratch_floats(int64_t n);                         // from the arena

    // ---- row-wise
    Tensor embedding(const int* tokens, int64_t n, const Tensor& table, Tensor* out = nullptr);
    Tensor gather_rows(const int* rows, int64_t n, const Tensor& src);
    Tensor rmsnorm(const Tensor& x, const Tensor& weight, float eps, Tensor* out = nullptr);
    Tensor swiglu(const Tensor& gate_up);                     // columns alternate gate, up
    // Rotates q and k inside qkv [rows, (nq + 2 nkv) * hd] (denominators null: no rotation) and, if the view
    // may be written, stores k and v in the cache rows of (row_seq, row_pos).
    void rope_kv_write(Tensor& qkv, const int* row_seq, const int* row_pos, const float* denominators, int rotary_dim,
                       int n_heads, int n_kv_heads, int head_dim, const CacheView* view);
    void advance(int* tokens, const int* sampled, int* row_pos, int* kv_len, const int* row_seq, int* draws, int n);
    void scale_rows(Tensor& x, float scale);                  // x *= scale (embedding multipliers)
    void finish_logits(Tensor& logits, const Tensor* bias, float scale, float softcap);

    // ---- matrix products: x [rows, k] @ weight [n, k]^T (+ bias [n]) (+ residual [rows, n])
    Tensor linear(const Rows& x, const Tensor& weight, const Tensor* bias = nullptr, const Tensor* residual = nullptr,
                  int out_dtype = -1, Tensor* out = nullptr);
    // linear(...) and the RMSNorm of its result.  For bf16 rows whose sizes allow it the norm is begun in the
    // product's epilogue and the second result is deferred; otherwise the norm's kernel runs.
    std::pair<Tensor, Rows> linear_norm(const Rows& x, const Tensor& weight, const Tensor& norm_weight, float eps,
                                        const Tensor* bias = nullptr, const Tensor* residual = nullptr);
    // linear(x, weight, bias) followed by rope_kv_write on its result; for up to 64 bf16 rows and a head size that
    // divides 128 both happen in the product's epilogue.
    Tensor qkv_rope_write(const Rows& x, const Tensor& weight, const Tensor* bias, const int* row_seq,
                          const int* row_pos, const float* denominators, int rotary_dim, int n_heads, int n_kv_heads,
                          int head_dim, const CacheView* view);
    // silu(x Wg^T) * (x Wu^T) for weight_pairs [2 * inner, k] whose rows alternate gate, up.
    Tensor linear_swiglu(const Rows& x, const Tensor& weight_pairs);
    Tensor materialize(const Rows& h);

    // ---- attention of the step's rows over the paged cache.  q: the buffer that holds the queries, row stride
    // q_stride elements, head h at h * head_dim.
    void attention(const Tensor& q, int64_t q_stride, Tensor& out, const CacheView& view, const StepContext& ctx,
                   int n_heads, int n_kv_heads, int head_dim, int window, float scale);

    // ---- sampling: one id per row of logits [rows, vocab] fp32
    void sample(const Tensor& logits, const float* temperature, const int* streams, const int* steps,
                unsigned long long seed, const int* row_live, int* out);

    // Raises KernelError if a kernel recorded that one of its bounded waits gave up (reads one word: call it
    // where the host waits for the device anyway); clears the word.
    void check_status();
    int* status_word() const { return (int*)status_.get(); }

    // ---- for tests and measurements
    Tensor linear_tc(const Tensor& x, const Tensor& weight, const Tensor* bias, const Tensor* residual, Tensor& out,
                     int swap = -1, int bn = -1, int splits = -1, int act = 0, GemmFusion* fusion = nullptr);
    Tensor linear_simt(const Tensor& x, const Tensor& weight, const Tensor* bias, const Tensor* residual, Tensor& out);
    bool tensor_core_ok(const Tensor& x, const Tensor& weight, const Tensor& out, const Tensor* residual) const;
    void plan(int64_t rows, int64_t n, int64_t k, bool* swapped, int* bn, int* splits = nullptr);
    int decode_splits(int n_seqs, int n_heads, int n_kv_heads, int head_dim, int max_kv_len);
    int attention_splits(int64_t rows, int n_heads, int max_kv_len) const;
    // FRIDAY_FUSE=0 keeps norms, rotation and cache write in kernels of their own (read at every call, for A/B runs)
    bool fusion_enabled() const;
    // For measurements: the next `launches` tensor-core products each fill one [sm_count][16] block of `trace`
    // (unsigned 64-bit) with their CTAs' time stamps (csrc/gemm_tc_fusion.h, part 4); null switches it off.
    void set_trace(unsigned long long* trace, int launches) { trace_ = trace; trace_left_ = launches; trace_next_ = 0; }
    long long launches() const { return launches_; }
    void add_launches(long long n) { launches_ += n; }

    // Event-bracketed time per kind of kernel (products, attention, everything else), switched on by
    // set_profile(true) or FRIDAY_PROFILE=1; read and cleared by take_profile (waits for the stream).
    enum Segment { Product = 0, Attention = 1, Other = 2, Segments = 3 };
    void set_profile(bool on);
    bool profiling() const { return profile_; }
    void take_profile(double ms[Segments], long long calls[Segments]);

private:
    struct Timed;
    friend struct Timed;
    bool few_rows_tile_ok(const Tensor& x, const Tensor& weight, const Tensor& out, const Tensor* residual,
                          int64_t max_rows, int columns = 128) const;
    void fusion_in(const Rows& x, GemmFusion& f) const;
    int device_, sms_;
    cudaStream_t stream_;
    DeviceBuffer tc_scratch_, tc_counters_, status_, attn_counters_;
    std::map<std::tuple<int64_t, int64_t, int64_t>, std::tuple<bool, int, int>> plans_;
    std::map<std::pair<int, int>, int> cluster_fit_;
    bool attn_tc_, profile_ = false;
    long long launches_ = 0;
    unsigned long long* trace_ = nullptr;
    int trace_left_ = 0, trace_next_ = 0;
    std::vector<std::tuple<int, cudaEvent_t, cudaEvent_t>> events_;
    std::vector<cudaEvent_t> spare_events_;
};

}  // namespace friday
