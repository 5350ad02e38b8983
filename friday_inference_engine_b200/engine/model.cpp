// DecoderModel: parts from a specification, weights from a source, one pass over rows (model.h).
#include "friday/model.h"

#include <set>

namespace friday {

class DecoderModel::Root : public Part {
public:
    explicit Root(const BuildEnv& e) : Part(e) {}
};

DecoderModel::DecoderModel(const ModelSpec& s, DType dtype) : spec(s) {
    env.width = s.width;
    env.dtype = dtype;
    if (s.vocab_size <= 0 || s.width <= 0) throw ConfigError("a model needs a vocabulary and a width");
    owners = spec.cache_entries();
    for (const auto& ls : spec.layers) layers.emplace_back(build<Block>("block", ls, env));
    final_norm.reset(build<Norm>("norm", spec.final_norm, env));
    root_.reset(new Root(env));
    root_->declare(spec.embedding, {spec.vocab_size, spec.width});
    if (!spec.head.empty()) root_->declare(spec.head, {spec.vocab_size, spec.width});
    if (!spec.head_bias.empty()) root_->declare(spec.head_bias, {spec.vocab_size});
}

std::vector<Part::Named> DecoderModel::named_params() {
    std::vector<Part::Named> out;
    root_->named_params("", out);
    for (size_t i = 0; i < layers.size(); ++i) layers[i]->named_params(spec.layers[i].prefix, out);
    final_norm->named_params(spec.final_norm.prefix, out);
    return out;
}

std::map<int, CacheRequest> DecoderModel::cache_requests() const {
    std::map<int, CacheRequest> out;
    for (const auto& kv : owners) out[kv.first] = layers[spec.program[kv.second].layer]->cache_request();
    return out;
}

static DType storage_dtype(const StoredTensor& st, const ParamDecl& d, DType compute, const std::string& name) {
    if (d.integer) return DType::I32;
    if (!stored_dtype_is_float(st.dtype))
        throw WeightsError("tensor '" + name + "': an integer tensor (" + st.dtype + ") where a floating one is needed");
    if (compute == DType::F32 || stored_dtype_is_32bit_float(st.dtype)) return DType::F32;
    return compute;
}

std::vector<StoredParam> plan_storage(const std::vector<Part::Named>& all, const WeightSource& source, DType compute,
                                      const std::vector<std::string>& ignorable) {
    std::vector<Part::Named> named;
    std::set<std::string> seen;
    for (auto& e : all)
        if (seen.insert(e.name).second) named.push_back(e);
    check_names(named, source, ignorable);
    std::vector<StoredParam> plan;
    // a stacked tensor is 32-bit if any member is stored so
    std::map<std::pair<Part*, std::string>, DType> stacked_dtype;
    for (const auto& e : named) {
        StoredTensor st;
        source.info(e.name, &st);
        StoredParam s;
        s.param = e;
        s.dtype = storage_dtype(st, e.decl, compute, e.name);
        if (!e.decl.into.empty()) {
            auto key = std::make_pair(e.owner, e.decl.into);
            auto it = stacked_dtype.find(key);
            if (it == stacked_dtype.end()) stacked_dtype[key] = s.dtype;
            else if (s.dtype == DType::F32) it->second = DType::F32;
        }
        plan.push_back(s);
    }
    for (auto& s : plan)
        if (!s.param.decl.into.empty()) s.dtype = stacked_dtype[std::make_pair(s.param.owner, s.param.decl.into)];
    return plan;
}

size_t load_params(const std::vector<StoredParam>& plan, WeightSource& source, Ops& ops) {
    size_t bytes = 0;
    for (const auto& s : plan) {          // stacked tensors first
        const Part::Named& e = s.param;
        if (e.decl.into.empty() || e.owner->tensors.count(e.decl.into)) continue;
        const std::vector<int64_t>* shape = nullptr;
        for (const auto& st : e.owner->stacked)
            if (st.first == e.decl.into) shape = &st.second;
        if (!shape) throw ConfigError("a parameter is stacked into '" + e.decl.into + "', which its part never declared");
        auto mem = std::make_shared<DeviceBuffer>((size_t)(*shape)[0] * (*shape)[1] * dtype_size(s.dtype));
        e.owner->set_tensor(e.decl.into, Tensor::make(mem->get(), s.dtype, *shape));
        e.owner->hold(mem);
        bytes += mem->bytes();
    }
    for (const auto& s : plan) {
        const Part::Named& e = s.param;
        Tensor dst;
        const int64_t cols = e.decl.shape.size() >= 2 ? e.decl.shape.back() : 1;
        if (e.decl.into.empty()) {
            int64_t n = 1;
            for (int64_t d : e.decl.shape) n *= d;
            auto mem = std::make_shared<DeviceBuffer>((size_t)n * dtype_size(s.dtype));
            Tensor t = Tensor::make(mem->get(), s.dtype, e.decl.shape);
            e.owner->set_tensor(e.local, t);
            e.owner->hold(mem);
            bytes += mem->bytes();
            dst = t;
            dst.ld = cols;
        } else {
            const Tensor& big = e.owner->tensor(e.decl.into);
            if (big.cols() != cols)
                throw ConfigError("parameter '" + e.name + "' does not have the columns of '" + e.decl.into + "' that it is stacked into");
            dst = big;
            dst.data = (char*)big.data + (size_t)e.decl.row0 * big.ld * dtype_size(big.dtype);
            dst.ld = big.ld * e.decl.row_step;
        }
        source.load(e.name, dst, ops.stream());
    }
    cuda_check(cudaStreamSynchronize(ops.stream()), "cudaStreamSynchronize");
    return bytes;
}

std::vector<StoredParam> DecoderModel::plan_storage(const WeightSource& source) {
    return friday::plan_storage(named_params(), source, env.dtype, spec.ignorable);
}

void DecoderModel::load(WeightSource& source, Ops& ops) {
    parameter_bytes_ = load_params(plan_storage(source), source, ops);
    embedding = root_->tensor(spec.embedding);
    head = spec.head.empty() ? embedding : root_->tensor(spec.head);       // tied: one copy in memory
    if (!spec.head_bias.empty()) head_bias = root_->tensor(spec.head_bias);
    for (auto& l : layers) l->finalize(ops);
    final_norm->finalize(ops);
}

DecoderModel::RunOut DecoderModel::run(Ops& ops, const StepContext& ctx, const std::vector<CacheView>& views,
                                       bool with_final_norm, Arena* layer_arenas[2]) {
    Arena* outer = ops.arena;
    Tensor x = ops.embedding(ctx.tokens, ctx.rows, embedding);
    if (spec.embed_scale != 1.0) ops.scale_rows(x, (float)spec.embed_scale);
    Rows normed;
    bool has_normed = false;
    const size_t n = spec.program.size();
    for (size_t i = 0; i < n; ++i) {
        const LayerCall& call = spec.program[i];
        Block* block = layers[call.layer].get();
        // the last entry's results must outlive the loop: they come from the caller's arena
        Arena* mine = (i + 1 == n) ? outer : layer_arenas[i & 1];
        if (mine != outer) mine->reset();
        ops.arena = mine;
        Norm* then = nullptr;
        if (i + 1 < n) then = layers[spec.program[i + 1].layer]->first_norm();
        else if (with_final_norm) then = final_norm.get();
        static const CacheView none;
        PartOut o = block->forward(ops, x, has_normed ? &normed : nullptr, ctx, call.cache >= 0 ? views[i] : none, then);
        x = o.x;
        has_normed = o.has_normed && then != nullptr;
        normed = o.normed;
    }
    ops.arena = outer;
    RunOut out;
    out.x = x;
    out.has_normed = has_normed && with_final_norm;
    out.normed = normed;
    return out;
}

Tensor DecoderModel::logits(Ops& ops, const Tensor& x, const int* rows, int64_t n_rows, const Rows* normed) {
    Rows h;
    if (rows) h = Rows(final_norm->forward(ops, ops.gather_rows(rows, n_rows, x)));
    else if (normed) h = *normed;
    else h = Rows(final_norm->forward(ops, x));
    Tensor out = ops.linear(h, head, nullptr, nullptr, (int)DType::F32);
    ops.finish_logits(out, head_bias.defined() ? &head_bias : nullptr, (float)spec.logit_scale, (float)spec.logit_softcap);
    return out;
}

}  // namespace friday
