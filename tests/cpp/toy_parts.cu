// A plug-in defined wholly in the tests: toy parts and a toy architecture registered from outside the library,
// and probes that build one shipped part alone and run it on tensors the test provides.
//
// Toy parts (none of them is anybody's model):
//   mixer "toy_running_mean"      out_t = W * mean(h_0 .. h_t): needs the sum so far and the count, a state of fixed
//                                 size per sequence, zero when a sequence starts
//   position "toy_additive"       not rotary: adds pos / 100 to the first dimension of every query and key head
//   feed_forward "toy_top1"       routing: a router picks one of a few small ReLU experts per row; the expert's output
//                                 is weighted with the router's probability for it (router logits in 32-bit)
// Toy architecture "ToyForCausalLM": Qwen2's keys; layer 1 has the toy mixer and the routed feed-forward, layer 2
// attention with the toy position; the run order names layer 0 twice (second time with a cache entry of its own) and
// lets the last call of layer 2 read the keys and values that its first call wrote; token rows are multiplied by
// 1.5, the head has a bias and the logits a multiplier.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <map>
#include <string>

#include "friday/capi.h"
#include "friday/config.h"
#include "friday/model.h"
#include "friday/ops.h"
#include "friday/parts.h"

using namespace friday;

namespace {

template <typename T> __device__ float ld(const T* p);
template <> __device__ float ld<float>(const float* p) { return *p; }
template <> __device__ float ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ void st(T* p, float v);
template <> __device__ void st<float>(float* p, float v) { *p = v; }
template <> __device__ void st<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// ---- running mean: one block per sequence, a scan over the sequence's rows in order, starting from the stored state
template <typename T>
__global__ void running_mean_kernel(const T* h, T* out, int width, const int* seq_start, const int* seq_qlen,
                                    const int* row_seq, const int* seq_slots, float* state) {
    const int seq = blockIdx.x, r0 = seq_start[seq], q = seq_qlen[seq];
    if (row_seq[r0] < 0) return;                                  // a sequence that has ended
    float* st_ = state + (size_t)seq_slots[seq] * (width + 1);
    const float count0 = st_[width];
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float sum = st_[c];
        for (int t = 0; t < q; ++t) {
            sum += ld(h + (size_t)(r0 + t) * width + c);
            st(out + (size_t)(r0 + t) * width + c, sum / (count0 + (float)(t + 1)));
        }
        st_[c] = sum;
    }
    __syncthreads();
    if (threadIdx.x == 0) st_[width] = count0 + (float)q;
}

class RunningMean : public Mixer {
public:
    RunningMean(const PartSpec&, const BuildEnv& e) : Mixer(e) { declare("mix.weight", {e.width, e.width}); }
    CacheRequest cache_request() const override { return CacheRequest::state({env.width + 1}, DType::F32); }
    PartOut forward(Ops& ops, const Rows& h, const Tensor& residual, const StepContext& ctx, const CacheView& view,
                    Norm*) override {
        Tensor x = ops.materialize(h);
        Tensor mean = ops.alloc(x.dtype, x.rows(), x.cols());
        if (x.dtype == DType::F32)
            running_mean_kernel<float><<<ctx.n_seqs, 128, 0, ops.stream()>>>(
                (const float*)x.data, (float*)mean.data, (int)x.cols(), ctx.seq_start, ctx.seq_qlen, ctx.row_seq,
                view.seq_slots, (float*)view.state.data);
        else
            running_mean_kernel<__nv_bfloat16><<<ctx.n_seqs, 128, 0, ops.stream()>>>(
                (const __nv_bfloat16*)x.data, (__nv_bfloat16*)mean.data, (int)x.cols(), ctx.seq_start, ctx.seq_qlen,
                ctx.row_seq, view.seq_slots, (float*)view.state.data);
        cuda_check(cudaGetLastError(), "running_mean_kernel");
        return PartOut(ops.linear(Rows(mean), tensor("mix.weight"), nullptr, &residual));
    }
};

// ---- additive position
template <typename T>
__global__ void additive_position_kernel(T* qkv, int64_t ld_, int heads, int head_dim, const int* row_pos, const int* row_seq) {
    const int row = blockIdx.x;
    if (row_seq[row] < 0) return;
    for (int hd = threadIdx.x; hd < heads; hd += blockDim.x) {
        T* p = qkv + (size_t)row * ld_ + (size_t)hd * head_dim;
        st(p, ld(p) + (float)row_pos[row] / 100.0f);
    }
}

class AdditivePosition : public Position {
public:
    AdditivePosition(const PartSpec&, const BuildEnv& e) : Position(e) {}
    void apply(Ops& ops, Tensor& qkv, const StepContext& ctx, int n_heads, int n_kv_heads, int head_dim) override {
        if (qkv.dtype == DType::F32)
            additive_position_kernel<float><<<(int)qkv.rows(), 64, 0, ops.stream()>>>(
                (float*)qkv.data, qkv.ld, n_heads + n_kv_heads, head_dim, ctx.row_pos, ctx.row_seq);
        else
            additive_position_kernel<__nv_bfloat16><<<(int)qkv.rows(), 64, 0, ops.stream()>>>(
                (__nv_bfloat16*)qkv.data, qkv.ld, n_heads + n_kv_heads, head_dim, ctx.row_pos, ctx.row_seq);
        cuda_check(cudaGetLastError(), "additive_position_kernel");
    }
};

// ---- routed experts: one block per row
template <typename T>
__global__ void top1_kernel(const T* h, const T* residual, T* out, int width, int experts, int inner, const T* router,
                            const T* up, const T* down) {
    extern __shared__ float sm[];
    float* logits = sm;                 // [experts]
    float* act = sm + experts;          // [inner]
    __shared__ int choice;
    __shared__ float prob;
    const int row = blockIdx.x;
    const T* x = h + (size_t)row * width;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        float s = 0.f;
        for (int c = 0; c < width; ++c) s += ld(x + c) * ld(router + (size_t)e * width + c);
        logits[e] = s;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int best = 0;
        for (int e = 1; e < experts; ++e)
            if (logits[e] > logits[best]) best = e;
        float total = 0.f;
        for (int e = 0; e < experts; ++e) total += expf(logits[e] - logits[best]);
        choice = best;
        prob = 1.0f / total;
    }
    __syncthreads();
    const T* u = up + (size_t)choice * inner * width;
    for (int i = threadIdx.x; i < inner; i += blockDim.x) {
        float s = 0.f;
        for (int c = 0; c < width; ++c) s += ld(x + c) * ld(u + (size_t)i * width + c);
        act[i] = fmaxf(s, 0.f);
    }
    __syncthreads();
    const T* d = down + (size_t)choice * width * inner;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float s = 0.f;
        for (int i = 0; i < inner; ++i) s += act[i] * ld(d + (size_t)c * inner + i);
        st(out + (size_t)row * width + c, ld(residual + (size_t)row * width + c) + s * prob);
    }
}

class Top1Experts : public FeedForward {
public:
    Top1Experts(const PartSpec& s, const BuildEnv& e) : FeedForward(e) {
        experts_ = (int)s.params.get_int("experts", 0);
        inner_ = (int)s.params.get_int("inner", 0);
        declare("router.weight", {experts_, e.width});
        declare("experts.up", {experts_, inner_, e.width});
        declare("experts.down", {experts_, e.width, inner_});
    }
    PartOut forward(Ops& ops, const Rows& h, const Tensor& residual, const StepContext&, Norm*) override {
        Tensor x = ops.materialize(h);
        Tensor out = ops.alloc(x.dtype, x.rows(), x.cols());
        const size_t smem = (size_t)(experts_ + inner_) * sizeof(float);
        if (x.dtype == DType::F32)
            top1_kernel<float><<<(int)x.rows(), 128, smem, ops.stream()>>>(
                (const float*)x.data, (const float*)residual.data, (float*)out.data, (int)x.cols(), experts_, inner_,
                (const float*)tensor("router.weight").data, (const float*)tensor("experts.up").data,
                (const float*)tensor("experts.down").data);
        else
            top1_kernel<__nv_bfloat16><<<(int)x.rows(), 128, smem, ops.stream()>>>(
                (const __nv_bfloat16*)x.data, (const __nv_bfloat16*)residual.data, (__nv_bfloat16*)out.data, (int)x.cols(),
                experts_, inner_, (const __nv_bfloat16*)tensor("router.weight").data,
                (const __nv_bfloat16*)tensor("experts.up").data, (const __nv_bfloat16*)tensor("experts.down").data);
        cuda_check(cudaGetLastError(), "top1_kernel");
        return PartOut(out);
    }

private:
    int experts_, inner_;
};

PartRegistrar t1("mixer", "toy_running_mean", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new RunningMean(s, e); });
PartRegistrar t2("position", "toy_additive", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new AdditivePosition(s, e); });
PartRegistrar t3("feed_forward", "toy_top1", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new Top1Experts(s, e); });

ModelSpec toy_spec(const Json& typed) {
    ModelSpec spec = qwen2_spec(typed);
    spec.architecture = "ToyForCausalLM";
    // layer 1: the toy mixer instead of attention, and routed experts
    PartSpec& l1 = spec.layers[1];
    l1.parts["mixer"] = PartSpec("toy_running_mean", Json::object(), "toy.");
    Json moe = Json::object();
    moe.set("experts", Json(3));
    moe.set("inner", Json(40));
    l1.parts["feed_forward"] = PartSpec("toy_top1", moe, "moe.");
    // layer 2: attention with the toy position encoding
    spec.layers[2].parts["mixer"].parts["position"] = PartSpec("toy_additive");
    // run order: 0, 1 (state), 2, then layer 0 AGAIN with a cache entry of its own, then layer 2 reading the keys
    // and values that the first call of layer 2 wrote
    spec.program.clear();
    const int order[5][3] = {{0, 0, 1}, {1, 1, 1}, {2, 2, 1}, {0, 3, 1}, {2, 2, 0}};
    for (const auto& o : order) {
        LayerCall c;
        c.layer = o[0];
        c.cache = o[1];
        c.write = o[2] != 0;
        spec.program.push_back(c);
    }
    spec.embed_scale = 1.5;
    spec.head_bias = "lm_head.bias";
    spec.logit_scale = 0.5;
    return spec;
}

struct RegisterToy {
    RegisterToy() { register_architecture({"ToyForCausalLM", Qwen2Config::read, toy_spec}); }
} register_toy;

// ------------------------------------------------------------------ probes: one part alone
thread_local std::string g_error, g_text;

#define PROBE(...)                           \
    try {                                    \
        __VA_ARGS__;                         \
        return 0;                            \
    } catch (const std::exception& x) {      \
        g_error = x.what();                  \
        return 1;                            \
    }

PartSpec spec_from(const Json& j) {
    PartSpec s(j.get_string("kind", ""), j.has("params") ? j.at("params") : Json::object(), j.get_string("prefix", ""));
    if (const Json* parts = j.find("parts"))
        for (const auto& m : parts->members()) s.parts[m.first] = spec_from(m.second);
    return s;
}

// tensors that the test provides on the device, already in the dtype they are to be kept in
class DeviceTensors : public WeightSource {
public:
    std::map<std::string, Tensor> tensors;
    std::vector<std::string> order;
    std::string where() const override { return "the test's tensors"; }
    std::vector<std::string> names() const override { return order; }
    bool info(const std::string& name, StoredTensor* out) const override {
        auto it = tensors.find(name);
        if (it == tensors.end()) return false;
        out->dtype = it->second.dtype == DType::BF16 ? "BF16" : it->second.dtype == DType::F32 ? "F32" : "I32";
        out->shape = it->second.dims();
        return true;
    }
    void load(const std::string& name, const Tensor& dst, cudaStream_t stream) override {
        const Tensor& t = tensors.at(name);
        if (t.dtype != dst.dtype) throw WeightsError("the probe's tensors must come in the dtype they are kept in");
        const int64_t cols = t.ndim >= 2 ? t.cols() : 1, rows = t.numel() / cols;
        const size_t es = dtype_size(t.dtype);
        cuda_check(cudaMemcpy2DAsync(dst.data, (size_t)dst.ld * es, t.data, (size_t)cols * es, (size_t)cols * es, (size_t)rows,
                                     cudaMemcpyDeviceToDevice, stream), "cudaMemcpy2DAsync");
    }
};

struct Probe {
    std::string category;
    std::unique_ptr<Part> part;
    std::unique_ptr<Ops> ops;
    std::unique_ptr<Arena> arena;
    Ops& begin() {
        arena->reset();
        ops->arena = arena.get();
        return *ops;
    }
};

Rows rows_of(const FridayTensor* x, const FridayTensor* ssq, float eps) {
    Rows r(*(const Tensor*)x);
    if (ssq && ssq->data) {
        r.deferred = true;
        r.ssq = *(const Tensor*)ssq;
        r.eps = eps;
    }
    return r;
}

void copy_out(Ops& ops, const Tensor& src, FridayTensor* dst) {
    const size_t es = dtype_size(src.dtype);
    cuda_check(cudaMemcpy2DAsync(dst->data, (size_t)dst->ld * es, src.data, (size_t)src.ld * es, (size_t)src.cols() * es,
                                 (size_t)src.rows(), cudaMemcpyDeviceToDevice, ops.stream()), "cudaMemcpy2DAsync");
}

// what a part returned beside its result when told which norm follows: 0 nothing, 1 a tensor, 2 deferred rows
int hand_normed(Ops& ops, const PartOut& o, FridayTensor* normed, FridayTensor* ssq) {
    if (!o.has_normed) return 0;
    copy_out(ops, o.normed.t, normed);
    if (!o.normed.deferred) return 1;
    ssq->shape[0] = o.normed.ssq.rows();
    copy_out(ops, o.normed.ssq, ssq);
    return 2;
}

}  // namespace

#define API extern "C" __attribute__((visibility("default")))

API const char* probe_error() { return g_error.c_str(); }

API int probe_new(const char* category, const char* spec_json, int64_t width, int dtype, void** handle) {
    PROBE({
        auto p = std::make_unique<Probe>();
        p->category = category;
        BuildEnv env;
        env.width = width;
        env.dtype = (DType)dtype;
        p->part.reset(build_part(category, spec_from(Json::parse(spec_json)), env));
        p->ops.reset(new Ops(0, nullptr));
        p->arena.reset(new Arena(nullptr));
        *handle = p.release();
    })
}
API void probe_free(void* h) { delete (Probe*)h; }

API int probe_params(void* h, const char** json) {
    PROBE({
        std::vector<Part::Named> named;
        ((Probe*)h)->part->named_params("", named);
        Json out = Json::array();
        for (const auto& n : named) {
            Json e = Json::object(), shape = Json::array();
            for (int64_t d : n.decl.shape) shape.push(Json(d));
            e.set("name", Json(n.name));
            e.set("shape", shape);
            e.set("one", Json(n.decl.one));
            out.push(e);
        }
        g_text = out.dump();
        *json = g_text.c_str();
    })
}

API int probe_load(void* h, int n, const char* const* names, const FridayTensor* tensors) {
    PROBE({
        Probe& p = *(Probe*)h;
        DeviceTensors src;
        for (int i = 0; i < n; ++i) {
            src.tensors[names[i]] = *(const Tensor*)&tensors[i];
            src.order.push_back(names[i]);
        }
        std::vector<Part::Named> named;
        p.part->named_params("", named);
        load_params(plan_storage(named, src, p.part->env.dtype, {}), src, *p.ops);
        p.part->finalize(*p.ops);
    })
}

// dtype and shape of a tensor the part holds after loading (a stacked one, for instance)
API int probe_tensor(void* h, const char* child_path, const char* name, FridayTensor* out) {
    PROBE({
        Part* part = ((Probe*)h)->part.get();
        std::string path = child_path;
        while (!path.empty()) {
            const size_t cut = path.find('/');
            const std::string head = path.substr(0, cut);
            Part* next = nullptr;
            for (const auto& c : part->children())
                if (c.first == head) next = c.second.get();
            if (!next) throw ConfigError("no child '" + head + "'");
            part = next;
            path = cut == std::string::npos ? "" : path.substr(cut + 1);
        }
        *(Tensor*)out = part->tensor(name);
    })
}

API int probe_norm(void* h, const FridayTensor* x, FridayTensor* out) {
    PROBE({
        Probe& p = *(Probe*)h;
        Norm* n = dynamic_cast<Norm*>(p.part.get());
        if (!n) throw ConfigError("not a norm");
        copy_out(*p.ops, n->forward(p.begin(), *(const Tensor*)x), out);
    })
}

API int probe_rotary(void* h, float* table_host, int* rotary_dim) {
    PROBE({
        Probe& p = *(Probe*)h;
        Position* pos = dynamic_cast<Position*>(p.part.get());
        if (!pos) throw ConfigError("not a position part");
        pos->finalize(*p.ops);
        const float* dev = nullptr;
        if (!pos->rotary(&dev, rotary_dim)) {
            *rotary_dim = -1;
            return 0;
        }
        cuda_check(cudaMemcpy(table_host, dev, (size_t)(*rotary_dim / 2) * sizeof(float), cudaMemcpyDeviceToHost), "cudaMemcpy");
    })
}

static StepContext context_of(const FridayGeometry* g) {
    StepContext ctx;
    ctx.rows = g->rows;
    ctx.n_seqs = g->n_seqs;
    ctx.max_q_len = g->max_q_len;
    ctx.max_kv_len = g->max_kv_len;
    ctx.decode = g->decode != 0;
    ctx.row_seq = g->row_seq;
    ctx.row_pos = g->row_pos;
    ctx.seq_start = g->seq_start;
    ctx.seq_qlen = g->seq_qlen;
    ctx.seq_pos0 = g->seq_pos0;
    return ctx;
}

API int probe_mixer(void* h, const FridayTensor* x, const FridayTensor* in_ssq, float in_eps, const FridayTensor* residual,
                    const FridayGeometry* g, const FridayKV* kv, void* then, FridayTensor* out, FridayTensor* normed,
                    FridayTensor* ssq, int* normed_kind) {
    PROBE({
        Probe& p = *(Probe*)h;
        Mixer* m = dynamic_cast<Mixer*>(p.part.get());
        if (!m) throw ConfigError("not a mixer");
        CacheView v;
        v.kind = CacheRequest::KV;
        v.k_pool = kv->k_pool;
        v.v_pool = kv->v_pool;
        v.pool_pages = kv->pool_pages;
        v.block_table = kv->block_table;
        v.table_width = kv->table_width;
        v.page_size = kv->page_size;
        v.window = kv->window;
        v.n_kv_heads = kv->n_kv_heads;
        v.head_dim = kv->head_dim;
        v.dtype = (DType)kv->dtype;
        v.write = kv->write != 0;
        Norm* norm = then ? dynamic_cast<Norm*>(((Probe*)then)->part.get()) : nullptr;
        Ops& ops = p.begin();
        PartOut o = m->forward(ops, rows_of(x, in_ssq, in_eps), *(const Tensor*)residual, context_of(g), v, norm);
        copy_out(ops, o.x, out);
        *normed_kind = hand_normed(ops, o, normed, ssq);
    })
}

API int probe_feed_forward(void* h, const FridayTensor* x, const FridayTensor* in_ssq, float in_eps,
                           const FridayTensor* residual, void* then, FridayTensor* out, FridayTensor* normed,
                           FridayTensor* ssq, int* normed_kind) {
    PROBE({
        Probe& p = *(Probe*)h;
        FeedForward* f = dynamic_cast<FeedForward*>(p.part.get());
        if (!f) throw ConfigError("not a feed-forward");
        Norm* norm = then ? dynamic_cast<Norm*>(((Probe*)then)->part.get()) : nullptr;
        Ops& ops = p.begin();
        StepContext ctx;
        ctx.rows = (int)x->shape[0];
        PartOut o = f->forward(ops, rows_of(x, in_ssq, in_eps), *(const Tensor*)residual, ctx, norm);
        copy_out(ops, o.x, out);
        *normed_kind = hand_normed(ops, o, normed, ssq);
    })
}
