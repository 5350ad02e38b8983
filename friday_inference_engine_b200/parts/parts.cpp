// The registry of parts, the description of a model as data, and the parts this library
// ships: RMSNorm, rotary NeoX encoding (and "none"), grouped-query attention, the SwiGLU
// feed-forward and the pre-norm residual block.
#include "friday/parts.h"

#include <dlfcn.h>
#include <math.h>

#include <mutex>

#include "friday/ops.h"

namespace friday {

// ------------------------------------------------------------------ specs
const PartSpec& PartSpec::part(const std::string& role) const {
    auto it = parts.find(role);
    if (it == parts.end()) throw ConfigError("part '" + kind + "' needs a sub-part '" + role + "' in its specification");
    return it->second;
}

std::map<int, int> ModelSpec::cache_entries() const {
    std::map<int, int> owners;
    for (size_t i = 0; i < program.size(); ++i) {
        const LayerCall& c = program[i];
        if (c.layer < 0 || c.layer >= (int)layers.size())
            throw ConfigError(format("program entry %zu names layer %d of %zu", i, c.layer, layers.size()));
        if (c.cache < 0 || !c.write) continue;
        if (owners.count(c.cache))
            throw ConfigError(format("cache entry %d is written by program entries %d and %zu", c.cache, owners[c.cache], i));
        owners[c.cache] = (int)i;
    }
    for (size_t i = 0; i < program.size(); ++i) {
        const LayerCall& c = program[i];
        if (c.cache >= 0 && !c.write && (!owners.count(c.cache) || owners[c.cache] > (int)i))
            throw ConfigError(format("program entry %zu reads cache entry %d before anything wrote it", i, c.cache));
    }
    return owners;
}

CacheRequest CacheRequest::kv(int n_kv_heads, int head_dim, int window) {
    CacheRequest r;
    r.kind = KV;
    r.n_kv_heads = n_kv_heads;
    r.head_dim = head_dim;
    r.window = window;
    return r;
}

CacheRequest CacheRequest::state(const std::vector<int64_t>& shape, DType dtype) {
    CacheRequest r;
    r.kind = State;
    r.state_shape = shape;
    r.state_dtype = dtype;
    return r;
}

// ------------------------------------------------------------------ Part
ParamDecl& Part::declare(const std::string& name, const std::vector<int64_t>& shape, bool integer, bool one) {
    ParamDecl d;
    d.shape = shape;
    d.integer = integer;
    d.one = one;
    params.emplace_back(name, d);
    return params.back().second;
}

const Tensor& Part::tensor(const std::string& name) const {
    auto it = tensors.find(name);
    if (it == tensors.end() || !it->second.defined())
        throw KernelError("part parameter '" + prefix + name + "' was never set (the model's weights are not loaded)");
    return it->second;
}

void Part::finalize(Ops& ops) {
    for (auto& c : children_) c.second->finalize(ops);
}

void Part::named_params(const std::string& pre, std::vector<Named>& out) {
    for (auto& p : params) out.push_back(Named{pre + p.first, this, p.first, p.second});
    for (auto& c : children_) c.second->named_params(pre + c.first, out);
}

// ------------------------------------------------------------------ registry
namespace {
const char* kCategories[] = {"norm", "position", "mixer", "feed_forward", "block"};
std::mutex& reg_mutex() { static std::mutex m; return m; }
std::map<std::string, std::map<std::string, PartFactory>>& reg() {
    static std::map<std::string, std::map<std::string, PartFactory>> r;
    return r;
}
bool known_category(const std::string& c) {
    for (const char* k : kCategories)
        if (c == k) return true;
    return false;
}
}  // namespace

void register_part(const std::string& category, const std::string& kind, PartFactory factory) {
    if (!known_category(category))
        throw ConfigError("unknown part category '" + category + "' (have: norm, position, mixer, feed_forward, block)");
    std::lock_guard<std::mutex> lock(reg_mutex());
    reg()[category][kind] = std::move(factory);
}

std::vector<std::string> registered_parts(const std::string& category) {
    if (!known_category(category))
        throw ConfigError("unknown part category '" + category + "' (have: norm, position, mixer, feed_forward, block)");
    std::lock_guard<std::mutex> lock(reg_mutex());
    std::vector<std::string> out;
    for (const auto& kv : reg()[category]) out.push_back(kv.first);
    return out;
}

Part* build_part(const std::string& category, const PartSpec& spec, const BuildEnv& env) {
    PartFactory f;
    {
        std::lock_guard<std::mutex> lock(reg_mutex());
        auto& kinds = reg()[category];
        auto it = kinds.find(spec.kind);
        if (it == kinds.end()) {
            std::string known;
            for (const auto& kv : kinds) known += (known.empty() ? "" : ", ") + kv.first;
            throw ConfigError("no " + category + " part named '" + spec.kind + "' (registered: " +
                              (known.empty() ? "none" : known) + ")");
        }
        f = it->second;
    }
    Part* p = f(spec, env);
    p->prefix = spec.prefix;
    return p;
}

void load_plugin(const std::string& path) {
    if (!dlopen(path.c_str(), RTLD_NOW | RTLD_GLOBAL))
        throw Error(ErrorKind::Other, "cannot load plug-in " + path + ": " + dlerror());
}

// ------------------------------------------------------------------ RMSNorm
// y = x / sqrt(mean(x^2) + eps) * weight, the mean taken in fp32.  Reference: rmsNormKernel
// (cuda_math_kernels.cu:280-321), friday_cpu::rmsNorm (cpu_ops.cpp:10-24).
class RMSNorm : public Norm {
public:
    RMSNorm(const PartSpec& s, const BuildEnv& e) : Norm(e) {
        const Json* eps = s.params.find("eps");
        if (!eps || !eps->is_number()) throw ConfigError("rmsnorm needs 'eps'");
        eps_ = (float)eps->as_double();
        width_ = s.params.get_int("width", e.width);
        declare("weight", {width_}, false, true);
    }
    Tensor forward(Ops& ops, const Tensor& x) override { return ops.rmsnorm(x, tensor("weight"), eps_); }
    bool as_rmsnorm(Tensor* weight, float* eps) const override {
        *weight = tensor("weight");
        *eps = eps_;
        return true;
    }

private:
    float eps_;
    int64_t width_;
};

// ------------------------------------------------------------------ rotary encoding, NeoX pairing
// The pair (i, i + rotary_dim/2) of every query and key head is rotated by the angle pos / theta^(2i / rotary_dim).
// The angle is formed as the reference forms it (cuda_math_kernels.cu:337-339, cpu_ops.cpp:26-30): the denominator
// theta^(2i/d) in fp32 (powf), then one fp32 division of the position by it.  The denominators are a table of
// rotary_dim/2 numbers, made once here; the kernel divides and takes sine and cosine per row.
class RotaryNeox : public Position {
public:
    RotaryNeox(const PartSpec& s, const BuildEnv& e) : Position(e) {
        theta_ = s.params.get_double("theta", 0);
        head_dim_ = (int)s.params.get_int("head_dim", 0);
        rotary_dim_ = (int)s.params.get_int("rotary_dim", head_dim_);
        if (theta_ <= 1.0) throw ConfigError("rotary_neox: 'theta' must be greater than 1");
        if (rotary_dim_ <= 0 || rotary_dim_ % 2 || rotary_dim_ > head_dim_)
            throw ConfigError(format("rotary_neox: rotary_dim %d must be even and at most head_dim %d", rotary_dim_, head_dim_));
        table_.resize(rotary_dim_ / 2);
        for (int i = 0; i < rotary_dim_ / 2; ++i)
            table_[i] = powf((float)theta_, (2.0f * (float)i) / (float)rotary_dim_);
    }
    void finalize(Ops& ops) override {
        Position::finalize(ops);
        auto mem = std::make_shared<DeviceBuffer>(table_.size() * sizeof(float));
        cuda_check(cudaMemcpyAsync(mem->get(), table_.data(), table_.size() * sizeof(float), cudaMemcpyHostToDevice, ops.stream()),
                   "cudaMemcpyAsync");
        cuda_check(cudaStreamSynchronize(ops.stream()), "cudaStreamSynchronize");
        denominators_ = (const float*)mem->get();
        hold(mem);
    }
    bool rotary(const float** denominators, int* rotary_dim) const override {
        *denominators = denominators_;
        *rotary_dim = rotary_dim_;
        return true;
    }
    const std::vector<float>& table() const { return table_; }

private:
    double theta_;
    int head_dim_, rotary_dim_;
    std::vector<float> table_;
    const float* denominators_ = nullptr;
};

// Leaves queries and keys as they are: not rotary, and apply() does nothing.
class NoPosition : public Position {
public:
    NoPosition(const PartSpec&, const BuildEnv& e) : Position(e) {}
};

// ------------------------------------------------------------------ grouped-query attention over the paged cache
// q = Wq h + bq, k = Wk h + bk, v = Wv h + bv (one product over the stacked matrices); q and k are encoded with the
// position part; k and v go to the cache at each row's (sequence, position); every query attends to the keys of its
// sequence up to its own position, or to the last `window` of them; the result goes through Wo and the residual is
// added in that product's epilogue.
//
// Reference order of operations: transformer.cpp:1013-1059 (norm is the block's), q/k/v bias in the product's
// epilogue (hpc_k_quants.cu:422-437), rotation and cache write in one kernel (cuda_math_kernels.cu:363-404),
// grouped heads h -> h / (heads / kv heads) and 1/sqrt(head_dim) scaling (attention_kernels.cu:45,
// cpu_ops.cpp:49-53), the output product with the residual (transformer.cpp:1057-1059).
class GQAttention : public Mixer {
public:
    GQAttention(const PartSpec& s, const BuildEnv& e) : Mixer(e) {
        nq_ = (int)s.params.get_int("n_heads", 0);
        nkv_ = (int)s.params.get_int("n_kv_heads", nq_);
        hd_ = (int)s.params.get_int("head_dim", 0);
        if (nq_ <= 0 || nkv_ <= 0 || hd_ <= 0) throw ConfigError("gqa_attention needs n_heads, n_kv_heads and head_dim");
        if (nq_ % nkv_) throw ConfigError(format("%d heads cannot share %d key/value heads", nq_, nkv_));
        window_ = (int)s.params.get_int("window", 0);
        scale_ = (float)s.params.get_double("scale", 1.0 / sqrt((double)hd_));
        qkv_bias_ = s.params.get_bool("qkv_bias", true);
        out_bias_ = s.params.get_bool("out_bias", false);
        position_ = adopt("", build<Position>("position", s.part("position"), e));
        const int64_t qd = (int64_t)nq_ * hd_, kvd = (int64_t)nkv_ * hd_, w = e.width;
        declare_stacked("w_qkv", qd + 2 * kvd, w);
        if (qkv_bias_) declare_stacked("b_qkv", qd + 2 * kvd, 1);      // a vector: one column, members under one another
        const char* names[3] = {"q_proj", "k_proj", "v_proj"};
        const int64_t rows[3] = {qd, kvd, kvd}, first[3] = {0, qd, qd + kvd};
        for (int i = 0; i < 3; ++i) {
            declare(std::string(names[i]) + ".weight", {rows[i], w}).stack("w_qkv", first[i]);
            if (qkv_bias_) declare(std::string(names[i]) + ".bias", {rows[i]}).stack("b_qkv", first[i]);
        }
        declare("o_proj.weight", {w, qd});
        if (out_bias_) declare("o_proj.bias", {w});
    }
    CacheRequest cache_request() const override { return CacheRequest::kv(nkv_, hd_, window_); }

    PartOut forward(Ops& ops, const Rows& h, const Tensor& residual, const StepContext& ctx, const CacheView& view,
                    Norm* then) override {
        const Tensor& w_qkv = tensor("w_qkv");
        Tensor bias_flat;
        const Tensor* b_qkv = nullptr;
        if (qkv_bias_) {
            const Tensor& b = tensor("b_qkv");
            bias_flat = Tensor::make(b.data, b.dtype, {b.numel()});
            b_qkv = &bias_flat;
        }
        const float* denominators = nullptr;
        int rotary_dim = 0;
        Tensor qkv;
        if (position_->rotary(&denominators, &rotary_dim)) {
            qkv = ops.qkv_rope_write(h, w_qkv, b_qkv, ctx.row_seq, ctx.row_pos, denominators, rotary_dim, nq_, nkv_, hd_, &view);
        } else {                                    // another encoding: it changes q and k itself
            qkv = ops.linear(h, w_qkv, b_qkv);
            position_->apply(ops, qkv, ctx, nq_, nkv_, hd_);
            if (view.write) ops.rope_kv_write(qkv, ctx.row_seq, ctx.row_pos, nullptr, 0, nq_, nkv_, hd_, &view);
        }
        Tensor mixed = ops.alloc(qkv.dtype, qkv.rows(), (int64_t)nq_ * hd_);
        ops.attention(qkv, qkv.ld, mixed, view, ctx, nq_, nkv_, hd_, window_, scale_);
        const Tensor& w_o = tensor("o_proj.weight");
        const Tensor* b_o = out_bias_ ? &tensor("o_proj.bias") : nullptr;
        Tensor nw;
        float eps;
        if (then && then->as_rmsnorm(&nw, &eps)) {
            auto r = ops.linear_norm(Rows(mixed), w_o, nw, eps, b_o, &residual);
            return PartOut(r.first, r.second);
        }
        return PartOut(ops.linear(Rows(mixed), w_o, b_o, &residual));
    }

private:
    int nq_, nkv_, hd_, window_;
    float scale_;
    bool qkv_bias_, out_bias_;
    Position* position_;
};

// ------------------------------------------------------------------ gated feed-forward: x + Wd (silu(Wg h) * (Wu h))
// Gate and up are one product, as the reference runs the two in one launch (transformer.cpp:1064-1066): their rows
// are stacked alternately (gate 0, up 0, gate 1, ...), so that every tile of the product holds both halves of a
// pair and silu(z) = z / (1 + e^-z) times up (cpu_ops.cpp:85-101, without its shortcuts for |z| > 20) can be
// applied in the product's epilogue; the residual is added in the down product's epilogue (transformer.cpp:1072).
class SwiGLU : public FeedForward {
public:
    SwiGLU(const PartSpec& s, const BuildEnv& e) : FeedForward(e) {
        inner_ = s.params.get_int("inner", 0);
        if (inner_ <= 0) throw ConfigError("swiglu needs 'inner'");
        declare_stacked("w_gate_up", 2 * inner_, e.width);
        declare("gate_proj.weight", {inner_, e.width}).stack("w_gate_up", 0, 2);
        declare("up_proj.weight", {inner_, e.width}).stack("w_gate_up", 1, 2);
        declare("down_proj.weight", {e.width, inner_});
    }
    PartOut forward(Ops& ops, const Rows& h, const Tensor& residual, const StepContext&, Norm* then) override {
        Tensor inner = ops.linear_swiglu(h, tensor("w_gate_up"));
        Tensor nw;
        float eps;
        if (then && then->as_rmsnorm(&nw, &eps)) {
            auto r = ops.linear_norm(Rows(inner), tensor("down_proj.weight"), nw, eps, nullptr, &residual);
            return PartOut(r.first, r.second);
        }
        return PartOut(ops.linear(Rows(inner), tensor("down_proj.weight"), nullptr, &residual));
    }

private:
    int64_t inner_;
};

// ------------------------------------------------------------------ pre-norm residual block
// x = x + mixer(norm1(x)); x = x + feed_forward(norm2(x)).  The two sums happen inside the mixer's and the
// feed-forward's last product (each gets the residual stream and returns it with its own output added), as in the
// reference (transformer.cpp:997-1074).  Which mixer, feed-forward and norms a block has is its specification's.
class PreNormBlock : public Block {
public:
    PreNormBlock(const PartSpec& s, const BuildEnv& e) : Block(e) {
        const PartSpec& n1 = s.part("norm1");
        const PartSpec& mx = s.part("mixer");
        const PartSpec& n2 = s.part("norm2");
        const PartSpec& ff = s.part("feed_forward");
        norm1_ = adopt(n1.prefix, build<Norm>("norm", n1, e));
        mixer_ = adopt(mx.prefix, build<Mixer>("mixer", mx, e));
        norm2_ = adopt(n2.prefix, build<Norm>("norm", n2, e));
        ffn_ = adopt(ff.prefix, build<FeedForward>("feed_forward", ff, e));
    }
    CacheRequest cache_request() const override { return mixer_->cache_request(); }
    Norm* first_norm() override { return norm1_; }

    PartOut forward(Ops& ops, const Tensor& x, const Rows* normed, const StepContext& ctx, const CacheView& view,
                    Norm* then) override {
        Rows h = normed ? *normed : Rows(norm1_->forward(ops, x));
        PartOut a = mixer_->forward(ops, h, x, ctx, view, norm2_);
        Rows h2 = a.has_normed ? a.normed : Rows(norm2_->forward(ops, a.x));
        PartOut b = ffn_->forward(ops, h2, a.x, ctx, then);
        if (then && !b.has_normed) {
            b.normed = Rows(then->forward(ops, b.x));
            b.has_normed = true;
        }
        return b;
    }

private:
    Norm *norm1_, *norm2_;
    Mixer* mixer_;
    FeedForward* ffn_;
};

namespace {
PartRegistrar r1("norm", "rmsnorm", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new RMSNorm(s, e); });
PartRegistrar r2("position", "rotary_neox", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new RotaryNeox(s, e); });
PartRegistrar r3("position", "none", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new NoPosition(s, e); });
PartRegistrar r4("mixer", "gqa_attention", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new GQAttention(s, e); });
PartRegistrar r5("feed_forward", "swiglu", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new SwiGLU(s, e); });
PartRegistrar r6("block", "prenorm", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new PreNormBlock(s, e); });
}  // namespace

}  // namespace friday
