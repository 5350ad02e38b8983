// The operations of ops.h: which kernel runs for which shapes, and what is fused into what.
//
// The choices follow what was measured on a B200: a bf16 product goes to the tcgen05
// kernel whenever its operands' rows start on 16-byte boundaries and to the CUDA-core
// kernel otherwise (and always in float32: the true 32-bit path uses no tensor cores);
// one-token steps let norms, rotation and the cache write ride in the products'
// epilogues; prompts' attention runs both products on tcgen05, one-token steps split
// the keys over the CTAs of a cluster.
#include "friday/ops.h"

#include <stdlib.h>
#include <string.h>

#include "ops/kernels.h"

namespace friday {

namespace {
inline int code(DType d) { return (int)d; }

bool env_on(const char* name, bool fallback = true) {
    const char* e = getenv(name);
    if (!e || !e[0]) return fallback;
    return e[0] != '0';
}

template <class K> void call(long long& launches, const K& k, int rc, const char* fn) {
    ++launches;
    if (rc != 0) throw KernelError(std::string(fn) + ": " + k.last_error());
}

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }
}  // namespace

struct Ops::Timed {
    Ops& ops;
    cudaEvent_t a = nullptr, b = nullptr;
    int seg;
    Timed(Ops& o, int s) : ops(o), seg(s) {
        if (!ops.profile_) return;
        auto take = [&]() {
            cudaEvent_t e;
            if (!ops.spare_events_.empty()) { e = ops.spare_events_.back(); ops.spare_events_.pop_back(); }
            else cuda_check(cudaEventCreate(&e), "cudaEventCreate");
            return e;
        };
        a = take();
        b = take();
        cudaEventRecord(a, ops.stream_);
    }
    ~Timed() {
        if (!a) return;
        cudaEventRecord(b, ops.stream_);
        ops.events_.emplace_back(seg, a, b);
    }
};

Ops::Ops(int device, cudaStream_t stream) : device_(device), stream_(stream) {
    cuda_check(cudaSetDevice(device), "cudaSetDevice");
    cudaDeviceProp prop;
    cuda_check(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
    sms_ = prop.multiProcessorCount;
    // Partial tiles of split-k (at most two tiles of 128 x 256 floats per CTA, one CTA per SM), tile counters, and
    // the word in which a kernel records a wait that gave up: made once, so that captured graphs keep their addresses.
    tc_scratch_ = DeviceBuffer((size_t)2 * sms_ * 128 * 256 * sizeof(float));
    tc_counters_ = DeviceBuffer(4096 * sizeof(int), true);
    status_ = DeviceBuffer(4 * sizeof(int), true);
    attn_counters_ = DeviceBuffer(((size_t)1 << 16) * sizeof(int), true);
    attn_tc_ = env_on("FRIDAY_ATTN_TC");
    profile_ = env_on("FRIDAY_PROFILE", false);
}

Ops::~Ops() {
    for (auto& e : events_) { cudaEventDestroy(std::get<1>(e)); cudaEventDestroy(std::get<2>(e)); }
    for (auto e : spare_events_) cudaEventDestroy(e);
}

void Ops::set_profile(bool on) { profile_ = on; }

bool Ops::fusion_enabled() const { return env_on("FRIDAY_FUSE"); }

void Ops::take_profile(double ms[Segments], long long calls[Segments]) {
    for (int i = 0; i < Segments; ++i) { ms[i] = 0; calls[i] = 0; }
    if (events_.empty()) return;
    cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
    for (auto& e : events_) {
        float t = 0;
        if (cudaEventElapsedTime(&t, std::get<1>(e), std::get<2>(e)) == cudaSuccess) {
            ms[std::get<0>(e)] += t;
            calls[std::get<0>(e)] += 1;
        }
        spare_events_.push_back(std::get<1>(e));
        spare_events_.push_back(std::get<2>(e));
    }
    events_.clear();
}

Tensor Ops::alloc(DType dtype, int64_t rows, int64_t cols) {
    if (!arena) throw KernelError("internal: an operation needs working memory and no arena is set");
    void* p = arena->alloc((size_t)rows * cols * dtype_size(dtype));
    return Tensor::make(p, dtype, {rows, cols});
}

float* Ops::scratch_floats(int64_t n) {
    if (!arena) throw KernelError("internal: an operation needs scratch memory and no arena is set");
    return (float*)arena->alloc((size_t)(n > 0 ? n : 1) * sizeof(float));
}

// ------------------------------------------------------------------ row-wise
Tensor Ops::embedding(const int* tokens, int64_t n, const Tensor& table, Tensor* out) {
    Tensor o = out ? *out : alloc(table.dtype, n, table.cols());
    const auto& k = kernels::rowwise();
    Timed t(*this, Other);
    call(launches_, k, k.embedding(tokens, table.data, o.data, (int)n, (int)table.cols(), (int)table.rows(), code(table.dtype), stream_),
         "embedding");
    return o;
}

Tensor Ops::gather_rows(const int* rows, int64_t n, const Tensor& src) {
    if (!src.contiguous()) throw KernelError("gather_rows: the source must be contiguous");
    Tensor o = alloc(src.dtype, n, src.cols());
    const auto& k = kernels::rowwise();
    Timed t(*this, Other);
    call(launches_, k, k.gather_rows(rows, src.data, o.data, (int)n, (int)src.cols(), code(src.dtype), stream_), "gather_rows");
    return o;
}

Tensor Ops::rmsnorm(const Tensor& x, const Tensor& weight, float eps, Tensor* out) {
    if (!x.contiguous() || weight.numel() != x.cols())
        throw KernelError(format("rmsnorm: rows of %lld columns (contiguous: %d), weight of %lld", (long long)x.cols(),
                                 (int)x.contiguous(), (long long)weight.numel()));
    Tensor o = out ? *out : alloc(x.dtype, x.rows(), x.cols());
    const auto& k = kernels::rowwise();
    Timed t(*this, Other);
    call(launches_, k, k.rmsnorm(x.data, weight.data, code(weight.dtype), o.data, (int)x.rows(), (int)x.cols(), eps,
                                 code(x.dtype), stream_), "rmsnorm");
    return o;
}

Tensor Ops::swiglu(const Tensor& gate_up) {
    if (!gate_up.contiguous() || gate_up.cols() % 2) throw KernelError("swiglu: rows must be contiguous pairs (gate, up)");
    const int64_t inner = gate_up.cols() / 2;
    Tensor o = alloc(gate_up.dtype, gate_up.rows(), inner);
    const auto& k = kernels::rowwise();
    Timed t(*this, Other);
    call(launches_, k, k.swiglu(gate_up.data, o.data, (int)gate_up.rows(), (int)inner, code(gate_up.dtype), stream_), "swiglu");
    return o;
}

void Ops::rope_kv_write(Tensor& qkv, const int* row_seq, const int* row_pos, const float* denominators, int rotary_dim,
                        int n_heads, int n_kv_heads, int head_dim, const CacheView* view) {
    if (!qkv.contiguous() || qkv.cols() != (int64_t)(n_heads + 2 * n_kv_heads) * head_dim)
        throw KernelError("rope_kv_write: qkv must be contiguous rows of (heads + 2 kv heads) * head_dim");
    const bool write = view && view->write && view->k_pool;
    if (write && view->dtype != qkv.dtype) throw KernelError("rope_kv_write: the cache's dtype differs from the rows'");
    const auto& k = kernels::rowwise();
    Timed t(*this, Other);
    call(launches_, k,
         k.rope_kv_write(qkv.data, row_seq, row_pos, denominators, denominators ? rotary_dim : 0, n_heads, n_kv_heads,
                         head_dim, write ? view->k_pool : nullptr, write ? view->v_pool : nullptr,
                         write ? view->block_table : nullptr, write ? view->table_width : 0,
                         view ? view->page_size : 0, write ? 1 : 0, (int)qkv.rows(), code(qkv.dtype), stream_),
         "rope_kv_write");
}

void Ops::advance(int* tokens, const int* sampled, int* row_pos, int* kv_len, const int* row_seq, int* draws, int n) {
    const auto& k = kernels::rowwise();
    Timed t(*this, Other);
    call(launches_, k, k.advance(tokens, sampled, row_pos, kv_len, row_seq, draws, n, stream_), "advance");
}

void Ops::scale_rows(Tensor& x, float scale) {
    if (scale == 1.0f) return;
    if (!x.contiguous()) throw KernelError("scale_rows: rows must be contiguous");
    const auto& k = kernels::rowwise();
    Timed t(*this, Other);
    call(launches_, k, k.scale_rows(x.data, (long long)x.numel(), scale, code(x.dtype), stream_), "scale_rows");
}

void Ops::finish_logits(Tensor& logits, const Tensor* bias, float scale, float softcap) {
    if (!bias && scale == 1.0f && softcap <= 0.f) return;
    if (logits.dtype != DType::F32) throw KernelError("finish_logits: logits are float32");
    if (bias && bias->numel() != logits.cols()) throw KernelError("finish_logits: the bias does not match the vocabulary");
    const auto& k = kernels::rowwise();
    Timed t(*this, Other);
    call(launches_, k, k.finish_logits((float*)logits.data, (int)logits.rows(), (int)logits.cols(), (int)logits.ld,
                                       bias ? bias->data : nullptr, bias ? code(bias->dtype) : 0, scale, softcap, stream_),
         "finish_logits");
}

// ------------------------------------------------------------------ matrix products
bool Ops::tensor_core_ok(const Tensor& x, const Tensor& weight, const Tensor& out, const Tensor* residual) const {
    (void)residual;
    return x.dtype == DType::BF16 && weight.dtype == DType::BF16 && (out.dtype == DType::BF16 || out.dtype == DType::F32) &&
           x.cols() % 8 == 0 && x.ld % 8 == 0 && weight.ld % 8 == 0 && aligned16(x.data) && aligned16(weight.data);
}

bool Ops::few_rows_tile_ok(const Tensor& x, const Tensor& weight, const Tensor& out, const Tensor* residual,
                           int64_t max_rows, int columns) const {
    return fusion_enabled() && out.dtype == DType::BF16 && x.rows() <= max_rows && weight.rows() % columns == 0 && out.ld % 8 == 0 &&
           aligned16(out.data) && (!residual || aligned16(residual->data)) && tensor_core_ok(x, weight, out, residual);
}

void Ops::fusion_in(const Rows& x, GemmFusion& f) const {
    if (!x.deferred) return;
    f.in_ssq = (const float*)x.ssq.data;
    f.in_parts = (int)x.ssq.rows();
    f.in_width = (float)x.t.cols();
    f.in_eps = x.eps;
}

void Ops::plan(int64_t rows, int64_t n, int64_t k, bool* swapped, int* bn, int* splits) {
    auto key = std::make_tuple(rows, n, k);
    auto it = plans_.find(key);
    if (it == plans_.end()) {
        long long p[8] = {0};
        const auto& g = kernels::gemm_tc();
        if (g.plan((int)rows, (int)n, (int)k, sms_, -1, -1, -1, p) != 0)
            throw KernelError(std::string("gemm_tc_plan: ") + g.last_error());
        if (plans_.size() > 4096) plans_.clear();
        it = plans_.emplace(key, std::make_tuple(p[0] != 0, (int)p[1], (int)p[2])).first;
    }
    if (swapped) *swapped = std::get<0>(it->second);
    if (bn) *bn = std::get<1>(it->second);
    if (splits) *splits = std::get<2>(it->second);
}

static void check_residual(const Tensor* residual, const Tensor& out) {
    if (!residual) return;
    if (residual->rows() != out.rows() || residual->cols() != out.cols() || residual->dtype != out.dtype ||
        residual->ld != out.ld)
        throw KernelError("linear: the residual must have the result's shape, dtype and row stride");
}

Tensor Ops::linear_tc(const Tensor& x, const Tensor& weight, const Tensor* bias, const Tensor* residual, Tensor& out,
                      int swap, int bn, int splits, int act, GemmFusion* fusion) {
    const auto& g = kernels::gemm_tc();
    Timed t(*this, Product);
    GemmFusion traced;
    if (trace_ && trace_next_ < trace_left_) {
        if (fusion) traced = *fusion;
        else memset(&traced, 0, sizeof traced);
        traced.trace = trace_ + (size_t)trace_next_++ * sms_ * 16;
        fusion = &traced;
    }
    call(launches_, g,
         g.fused(x.data, weight.data, out.data, code(out.dtype), bias ? bias->data : nullptr, bias ? code(bias->dtype) : 0,
                 residual ? residual->data : nullptr, (int)x.rows(), (int)weight.rows(), (int)x.cols(), (int)x.ld,
                 (int)weight.ld, (int)out.ld, (float*)tc_scratch_.get(), (long long)(tc_scratch_.bytes() / sizeof(float)),
                 (int*)tc_counters_.get(), (int)(tc_counters_.bytes() / sizeof(int)), (int*)status_.get(), sms_, swap, bn,
                 splits, act, fusion, stream_),
         "gemm_tc_fused");
    return out;
}

Tensor Ops::linear_simt(const Tensor& x, const Tensor& weight, const Tensor* bias, const Tensor* residual, Tensor& out) {
    const auto& g = kernels::gemm_simt();
    Timed t(*this, Product);
    call(launches_, g,
         g.gemm(x.data, code(x.dtype), weight.data, code(weight.dtype), out.data, code(out.dtype),
                bias ? bias->data : nullptr, bias ? code(bias->dtype) : 0, residual ? residual->data : nullptr,
                (int)x.rows(), (int)weight.rows(), (int)x.cols(), (int)x.ld, (int)weight.ld, (int)out.ld, stream_),
         "gemm_simt");
    return out;
}

static void check_product(const Tensor& x, const Tensor& weight) {
    if (x.ndim != 2 || weight.ndim != 2)
        throw KernelError("linear: input and weight must be 2-d");
    if (weight.cols() != x.cols())
        throw KernelError(format("linear: input has %lld columns, weight is [%lld, %lld]", (long long)x.cols(),
                                 (long long)weight.rows(), (long long)weight.cols()));
}

Tensor Ops::linear(const Rows& x, const Tensor& weight, const Tensor* bias, const Tensor* residual, int out_dtype,
                   Tensor* out) {
    const Tensor& xt = x.t;
    check_product(xt, weight);
    const DType od = out_dtype < 0 ? xt.dtype : (DType)out_dtype;
    Tensor o = out ? *out : alloc(od, xt.rows(), weight.rows());
    check_residual(residual, o);
    if (tensor_core_ok(xt, weight, o, residual)) {
        GemmFusion f;
        memset(&f, 0, sizeof f);
        fusion_in(x, f);
        return linear_tc(xt, weight, bias, residual, o, -1, -1, -1, 0, x.deferred ? &f : nullptr);
    }
    Tensor xin = x.deferred ? materialize(x) : xt;
    return linear_simt(xin, weight, bias, residual, o);
}

Tensor Ops::materialize(const Rows& h) {
    return h.deferred ? rmsnorm(h.source, h.weight, h.eps) : h.t;
}

std::pair<Tensor, Rows> Ops::linear_norm(const Rows& x, const Tensor& weight, const Tensor& norm_weight, float eps,
                                         const Tensor* bias, const Tensor* residual) {
    const Tensor& xt = x.t;
    check_product(xt, weight);
    const int64_t rows = xt.rows(), n = weight.rows();
    if (norm_weight.numel() == n) {
        Tensor probe = Tensor::make((void*)16, xt.dtype, {rows, n});      // shape and alignment of a fresh result
        // few rows: the weights lie on the tiles' M side (the planner's choice up to 128 rows) and every tile of 128
        // columns adds one partial sum per row; many rows: the rows lie on the M side and every column tile adds one
        bool few = false, many = false;
        int bn = 0, swap = -1;
        if (tensor_core_ok(xt, weight, probe, residual)) {
            bool swapped = false;
            plan(rows, n, xt.cols(), &swapped, &bn);
            few = swapped && few_rows_tile_ok(xt, weight, probe, residual, 128);
            many = !few && n % 16 == 0 && few_rows_tile_ok(xt, weight, probe, residual, rows, 16);
            if (many && swapped) {
                // few rows whose width is no multiple of 128: the fused norm wants whole tiles that way round, so the
                // product runs the other way round
                long long p[8] = {0};
                const auto& g = kernels::gemm_tc();
                if (g.plan((int)rows, (int)n, (int)xt.cols(), sms_, 0, -1, -1, p) != 0)
                    throw KernelError(std::string("gemm_tc_plan: ") + g.last_error());
                bn = (int)p[1];
                swap = 0;
            }
        }
        if (few || many) {
            Tensor out = alloc(xt.dtype, rows, n);
            check_residual(residual, out);
            Tensor scaled = alloc(xt.dtype, rows, n);
            const int64_t parts = few ? n / 128 : (n + bn - 1) / bn;
            Tensor ssq = alloc(DType::F32, parts, rows);
            GemmFusion f;
            memset(&f, 0, sizeof f);
            fusion_in(x, f);
            f.norm_w = norm_weight.data;
            f.norm_w_dtype = code(norm_weight.dtype);
            f.norm_out = scaled.data;
            f.out_ssq = (float*)ssq.data;
            linear_tc(xt, weight, bias, residual, out, swap, -1, -1, 0, &f);
            Rows r;
            r.t = scaled;
            r.deferred = true;
            r.ssq = ssq;
            r.eps = eps;
            r.source = out;
            r.weight = norm_weight;
            return {out, r};
        }
    }
    Tensor out = linear(x, weight, bias, residual);
    return {out, Rows(rmsnorm(out, norm_weight, eps))};
}

Tensor Ops::qkv_rope_write(const Rows& x, const Tensor& weight, const Tensor* bias, const int* row_seq,
                           const int* row_pos, const float* denominators, int rotary_dim, int n_heads, int n_kv_heads,
                           int head_dim, const CacheView* view) {
    const Tensor& xt = x.t;
    check_product(xt, weight);
    const int64_t n = weight.rows();
    const bool write = view && view->write && view->k_pool;
    if (128 % head_dim == 0 && head_dim % 8 == 0 && n == (int64_t)(n_heads + 2 * n_kv_heads) * head_dim &&
        (!denominators || rotary_dim % 16 == 0)) {
        Tensor probe = Tensor::make((void*)16, xt.dtype, {xt.rows(), n});
        if (few_rows_tile_ok(xt, weight, probe, nullptr, 64) && (!write || view->dtype == DType::BF16)) {
            Tensor out = alloc(xt.dtype, xt.rows(), n);
            GemmFusion f;
            memset(&f, 0, sizeof f);
            fusion_in(x, f);
            f.row_seq = row_seq;
            f.row_pos = row_pos;
            f.denom = denominators;
            f.rot = denominators ? rotary_dim : 0;
            f.nq = n_heads;
            f.nkv = n_kv_heads;
            f.hd = head_dim;
            if (write) {
                f.k_pool = view->k_pool;
                f.v_pool = view->v_pool;
                f.table = view->block_table;
                f.table_width = view->table_width;
                f.page = view->page_size;
            }
            return linear_tc(xt, weight, bias, nullptr, out, -1, -1, -1, 0, &f);
        }
    }
    Tensor qkv = linear(x, weight, bias);
    if (denominators || write) rope_kv_write(qkv, row_seq, row_pos, denominators, rotary_dim, n_heads, n_kv_heads, head_dim, view);
    return qkv;
}

Tensor Ops::linear_swiglu(const Rows& x, const Tensor& weight_pairs) {
    const Tensor& xt = x.t;
    check_product(xt, weight_pairs);
    const int64_t inner = weight_pairs.rows() / 2;
    Tensor probe = Tensor::make((void*)16, xt.dtype, {xt.rows(), inner});
    if (xt.dtype == DType::BF16 && tensor_core_ok(xt, weight_pairs, probe, nullptr)) {
        Tensor out = alloc(xt.dtype, xt.rows(), inner);
        GemmFusion f;
        memset(&f, 0, sizeof f);
        fusion_in(x, f);
        return linear_tc(xt, weight_pairs, nullptr, nullptr, out, -1, -1, -1, 1, x.deferred ? &f : nullptr);
    }
    return swiglu(linear(x, weight_pairs));
}

// ------------------------------------------------------------------ attention
int Ops::attention_splits(int64_t rows, int n_heads, int max_kv_len) const {
    // CUDA-core kernel: few rows facing long contexts are cut along the keys so that the device fills.
    const int64_t warps = rows * n_heads, want = (int64_t)sms_ * 16;
    if (warps >= want || max_kv_len <= 128) return 1;
    int64_t s = want / (warps > 0 ? warps : 1);
    const int64_t blocks = (max_kv_len + 63) / 64;
    if (s > blocks) s = blocks;
    if (s > 64) s = 64;
    return (int)(s < 1 ? 1 : s);
}

// FRIDAY_ATTN_WIDE=0: the CTAs that share a sequence's keys in a one-token step always form one thread-block cluster.
static bool wide_splits() {
    const char* e = getenv("FRIDAY_ATTN_WIDE");
    return e == nullptr || e[0] != '0';
}

int Ops::decode_splits(int n_seqs, int n_heads, int n_kv_heads, int head_dim, int max_kv_len) {
    // How many CTAs share one sequence's keys in a one-token step: the number with the shortest estimated time.
    // Up to 8 they form a thread-block cluster and merge through each other's shared memory; 9 to 64 leave partial
    // rows in memory and the last to finish merges them.  The estimate, in us, fitted to one-token steps of 1 to 32
    // sequences with 2,000 to 32,000 keys on a B200 (28 query heads on 4 kv heads of 128):
    //  - a CTA streams a block of 64 keys in 0.84 us while it has its SM to itself; the more SMs hold two CTAs, the
    //    slower each gets (1.13 us when 108 of 148 SMs hold two);
    //  - the device says how many clusters of a size it holds when empty; SMs that the kernel before frees one by
    //    one are packed less well, the worse the larger the cluster (32 clusters of 8 ran in two waves although 33
    //    fit, 32 of 7 were slower than 32 of 6 although 37 fit), so 2 % less per CTA of a cluster count as one wave,
    //    and every wave costs its CTAs' set-up and the merge again (2.5 us and 0.15 us per CTA of a cluster; through
    //    memory 5 us and 0.2 us per CTA).
    const int group = n_heads / n_kv_heads;
    const long long base = (long long)n_seqs * n_kv_heads * ((group + 15) / 16);
    if (base < 1) return 1;
    if (const char* e = getenv("FRIDAY_ATTN_SPLITS")) {              // for measurements: this many, whatever the shape
        const int v = atoi(e);
        if (v >= 1 && v <= 64) return v;
    }
    const int blocks = (max_kv_len + 63) / 64;
    int top = blocks / 2 < 1 ? 1 : blocks / 2;                      // every CTA keeps at least two blocks
    if (top > 8) top = 8;
    auto fit_of = [&](int size) {
        auto key = std::make_pair(head_dim, size);
        auto it = cluster_fit_.find(key);
        if (it == cluster_fit_.end()) it = cluster_fit_.emplace(key, kernels::attention_mma().clusters_at_once(head_dim, size)).first;
        return (long long)((1.0 - 0.02 * size) * it->second);
    };
    auto per_block = [&](double resident) {
        const double second = resident > sms_ ? resident - sms_ : 0.0;
        return 0.84 * (1.0 + 0.47 * second / sms_);
    };
    double best = 1e30;
    int pick = 1;
    for (int size = 1; size <= top; ++size) {
        const long long fit = fit_of(size);
        if (fit < 1) continue;
        const int per = (blocks + size - 1) / size;
        double t = 0.0;
        for (long long left = base; left > 0;) {
            const long long now = left < fit ? left : fit;
            t += per * per_block((double)now * size) + 2.5 + 0.15 * size;
            left -= now;
        }
        if (t < best) {
            best = t;
            pick = size;
        }
    }
    if (wide_splits()) {
        const long long at_once = fit_of(1);
        for (int wide = 9; wide <= 64 && wide <= blocks / 3 && base * wide <= at_once; ++wide) {
            const double t = (blocks + wide - 1) / wide * per_block((double)base * wide) + 5.0 + 0.2 * wide;
            if (t < best) {
                best = t;
                pick = wide;
            }
        }
    }
    return pick;
}

void Ops::attention(const Tensor& q, int64_t q_stride, Tensor& out, const CacheView& view, const StepContext& ctx,
                    int n_heads, int n_kv_heads, int head_dim, int window, float scale) {
    if (view.kind != CacheRequest::KV || !view.k_pool) throw KernelError("attention needs a view of keys and values");
    const bool geometry = ctx.seq_start != nullptr;
    const bool hd_ok = head_dim % 16 == 0 && head_dim >= 16 && head_dim <= 128 && view.page_size == 64;
    const int rows = (int)out.rows();
    if (out.dtype == DType::BF16 && geometry && !ctx.decode && attn_tc_ && hd_ok && n_kv_heads > 0 &&
        n_heads % n_kv_heads == 0 && n_heads / n_kv_heads <= 128 && q_stride % 8 == 0) {
        const auto& k = kernels::attention_tc();
        Timed t(*this, Attention);
        call(launches_, k,
             k.run(q.data, (int)q_stride, (int)q.rows(), out.data, view.k_pool, view.v_pool, view.pool_pages,
                   view.block_table, view.table_width, ctx.seq_start, ctx.seq_qlen, ctx.seq_pos0, ctx.row_seq, ctx.n_seqs,
                   ctx.max_q_len, n_heads, n_kv_heads, head_dim, window, scale, (int*)status_.get(), stream_),
             "attention_tc");
        return;
    }
    if (out.dtype == DType::BF16 && geometry && hd_ok) {
        const bool keys_mode = ctx.decode;
        const int splits = keys_mode ? decode_splits(ctx.n_seqs, n_heads, n_kv_heads, head_dim, ctx.max_kv_len) : 1;
        float* scratch = splits > 1 ? scratch_floats((int64_t)rows * n_heads * splits * (head_dim + 2)) : nullptr;
        const auto& k = kernels::attention_mma();
        Timed t(*this, Attention);
        call(launches_, k,
             k.run(q.data, (int)q_stride, out.data, view.k_pool, view.v_pool, view.pool_pages, view.block_table,
                   view.table_width, 64, ctx.seq_start, ctx.seq_qlen, ctx.seq_pos0, ctx.row_seq, ctx.n_seqs, rows,
                   ctx.max_q_len, n_heads, n_kv_heads, head_dim, window, scale, keys_mode ? 1 : 0, splits, scratch,
                   (int*)attn_counters_.get(), (int)(attn_counters_.bytes() / sizeof(int)), (int*)status_.get(), stream_),
             "attention_mma");
        return;
    }
    const int splits = attention_splits(rows, n_heads, ctx.max_kv_len);
    float* scratch = splits > 1 ? scratch_floats((int64_t)rows * n_heads * splits * (head_dim + 2)) : nullptr;
    const auto& k = kernels::attention_simt();
    Timed t(*this, Attention);
    call(launches_, k,
         k.run(q.data, (int)q_stride, out.data, view.k_pool, view.v_pool, view.block_table, view.table_width,
               view.page_size, ctx.row_seq, ctx.row_pos, rows, n_heads, n_kv_heads, head_dim, window, scale, splits,
               scratch, code(out.dtype), stream_),
         "attention_simt");
}

// ------------------------------------------------------------------ sampling
void Ops::sample(const Tensor& logits, const float* temperature, const int* streams, const int* steps,
                 unsigned long long seed, const int* row_live, int* out) {
    if (logits.dtype != DType::F32) throw KernelError("sample: logits are float32");
    const auto& k = kernels::sampling();
    Timed t(*this, Other);
    call(launches_, k,
         k.sample((const float*)logits.data, (int)logits.rows(), (int)logits.cols(), (int)logits.ld, temperature, streams,
                  steps, seed, row_live, out, stream_),
         "sampling_sample");
}

void Ops::check_status() {
    int word[4] = {0, 0, 0, 0};
    cuda_check(cudaMemcpyAsync(word, status_.get(), sizeof word, cudaMemcpyDeviceToHost, stream_), "cudaMemcpyAsync");
    cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
    if (word[0] != 0) {
        cuda_check(cudaMemsetAsync(status_.get(), 0, sizeof word, stream_), "cudaMemsetAsync");
        throw KernelError(format("a tensor-core kernel on device %d gave up waiting (code %d: which of its bounded waits, "
                                 "see gemm_tc.cu and attention_tc.cu); its results are not valid", device_, word[0]));
    }
}

}  // namespace friday
