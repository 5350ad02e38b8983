// friday::Engine (engine.h): construction from a model folder or a configuration, the step function, the
// single-sequence conveniences, generation, and the profile counters.
#include <string.h>

#include <algorithm>
#include <numeric>
#include <set>

#include "engine/engine_impl.h"
#include "friday/sampling.h"
#include "ops/kernels.h"

namespace friday {

// ------------------------------------------------------------------ pinned staging
PinnedRing::~PinnedRing() {
    for (auto& s : slots_) {
        if (s.ev) cudaEventDestroy(s.ev);
        if (s.p) cudaFreeHost(s.p);
    }
}

void* PinnedRing::next(size_t bytes) {
    Slot& s = slots_[next_ % 4];
    last_ = next_ % 4;
    ++next_;
    if (s.busy) {
        cuda_check(cudaEventSynchronize(s.ev), "cudaEventSynchronize");       // the copy that last used this buffer is done
        s.busy = false;
    }
    if (s.cap < bytes) {
        if (s.p) cudaFreeHost(s.p);
        s.cap = std::max(bytes, (size_t)16384);
        cuda_check(cudaMallocHost(&s.p, s.cap), "cudaMallocHost");
    }
    return s.p;
}

void PinnedRing::sent(cudaStream_t stream) {
    Slot& s = slots_[last_];
    if (!s.ev) cuda_check(cudaEventCreateWithFlags(&s.ev, cudaEventDisableTiming), "cudaEventCreate");
    cuda_check(cudaEventRecord(s.ev, stream), "cudaEventRecord");
    s.busy = true;
}

// ------------------------------------------------------------------ the step function
Stepper::Stepper(DecoderModel& model, Cache& cache, Ops& ops, int chunk)
    : model_(model), cache_(cache), ops_(ops), chunk_(chunk > 0 ? chunk : 2560), pass_(ops.stream()),
      layer_a_(ops.stream()), layer_b_(ops.stream()), keep_(ops.stream()) {}

void Stepper::check(const StepBatch& b) const {
    const size_t n = b.slots.size();
    if (n == 0) throw StepError("a step needs at least one sequence");
    if (b.tokens.size() != n || b.want.size() != n) throw StepError("slots, tokens and want must have one item per sequence");
    std::vector<int> sorted = b.slots;
    std::sort(sorted.begin(), sorted.end());
    if (std::adjacent_find(sorted.begin(), sorted.end()) != sorted.end()) throw StepError("a sequence appears twice in one step");
    const int limit = std::min<int64_t>(cache_.max_seq_tokens, model_.spec.max_positions);
    const int vocab = (int)model_.spec.vocab_size;
    for (size_t i = 0; i < n; ++i) {
        const auto& toks = b.tokens[i];
        if (toks.empty()) throw StepError("a sequence in a step brings no token");
        if (!cache_.slots.holds(b.slots[i])) throw StepError(format("slot %d is not held", b.slots[i]));
        for (int t : toks)
            if (t < 0 || t >= vocab) throw StepError(format("token id %d is outside the vocabulary [0, %d)", t, vocab));
        const int have = cache_.lens[b.slots[i]];
        if (have + (int)toks.size() > limit)
            throw StepError(format("context length exceeded: the sequence would hold %d tokens, the limit is %d",
                                   have + (int)toks.size(), limit));
        for (int p : b.want[i])
            if (p < 0 || p >= (int)toks.size())
                throw StepError(format("logits wanted at place %d of %zu tokens", p, toks.size()));
    }
}

static inline size_t pad4(size_t n) { return (n + 3) & ~(size_t)3; }

size_t Stepper::step(const StepBatch& b, float* out, bool out_on_device) {
    const auto t_begin = std::chrono::steady_clock::now();
    check(b);
    const size_t n = b.slots.size();
    const int64_t vocab = model_.spec.vocab_size;
    size_t total_want = 0;
    for (const auto& w : b.want) total_want += w.size();
    keep_.reset();
    // the result, in the order of the sequences and of `want`: rows are scattered here pass by pass
    Tensor result;
    if (total_want) result = Tensor::make(keep_.alloc(total_want * vocab * sizeof(float)), DType::F32, {(int64_t)total_want, vocab});
    std::vector<size_t> want_base(n, 0);
    for (size_t i = 1; i < n; ++i) want_base[i] = want_base[i - 1] + b.want[i - 1].size();
    std::vector<int> done(n, 0);
    Arena* layer_arenas[2] = {&layer_a_, &layer_b_};
    while (true) {
        std::vector<int> live;
        for (size_t i = 0; i < n; ++i)
            if (done[i] < (int)b.tokens[i].size()) live.push_back((int)i);
        if (live.empty()) break;
        // this pass's pieces
        std::vector<int> slots, q_lens, start;
        int rows = 0;
        for (int i : live) {
            // what is left of the sequence in passes of equal size (whole pages), none longer than the chunk: a last
            // pass of a few hundred tokens would fill the device badly
            const int left = (int)b.tokens[i].size() - done[i];
            const int passes = (left + chunk_ - 1) / chunk_;
            const int even = ((left + passes - 1) / passes + PAGE - 1) / PAGE * PAGE;
            const int q = std::min(left, std::min(chunk_, even));
            slots.push_back(b.slots[i]);
            q_lens.push_back(q);
            start.push_back(cache_.lens[b.slots[i]]);
            rows += q;
        }
        std::vector<int> want_rows;            // rows of this pass whose logits are wanted ...
        std::vector<size_t> want_dest;         // ... and the row of the result each goes to
        {
            int base = 0;
            for (size_t k = 0; k < live.size(); ++k) {
                const int i = live[k];
                for (size_t wi = 0; wi < b.want[i].size(); ++wi) {
                    const int p = b.want[i][wi];
                    if (p >= done[i] && p < done[i] + q_lens[k]) {
                        want_rows.push_back(base + p - done[i]);
                        want_dest.push_back(want_base[i] + wi);
                    }
                }
                base += q_lens[k];
            }
        }
        cache_.reserve(slots, q_lens);
        const size_t nseq = live.size(), nwant = want_rows.size();
        const size_t n_groups = cache_.groups.size();
        std::vector<size_t> sizes = {(size_t)rows, (size_t)rows, (size_t)rows, nwant, nseq, nseq, nseq, nseq};
        for (size_t g = 0; g < n_groups; ++g) sizes.push_back(nseq * cache_.groups[g]->width);
        std::vector<size_t> offs(sizes.size() + 1, 0);
        for (size_t i = 0; i < sizes.size(); ++i) offs[i + 1] = offs[i] + pad4(sizes[i]);
        const size_t ints = offs.back();
        int* host = (int*)ring_.next(ints * sizeof(int));
        {
            int r = 0;
            for (size_t k = 0; k < nseq; ++k) {
                const int i = live[k];
                for (int t = 0; t < q_lens[k]; ++t, ++r) {
                    host[offs[0] + r] = b.tokens[i][done[i] + t];
                    host[offs[1] + r] = (int)k;
                    host[offs[2] + r] = start[k] + t;
                }
                host[offs[4] + k] = r - q_lens[k];
                host[offs[5] + k] = q_lens[k];
                host[offs[6] + k] = start[k];
                host[offs[7] + k] = slots[k];
            }
            for (size_t w = 0; w < nwant; ++w) host[offs[3] + w] = want_rows[w];
            std::vector<int> rowsbuf;
            for (size_t g = 0; g < n_groups; ++g) {
                rowsbuf.clear();
                cache_.table_rows((int)g, slots, rowsbuf);
                memcpy(host + offs[8 + g], rowsbuf.data(), rowsbuf.size() * sizeof(int));
            }
        }
        pass_.reset();
        ops_.arena = &pass_;
        int* dev = (int*)pass_.alloc(ints * sizeof(int));
        cuda_check(cudaMemcpyAsync(dev, host, ints * sizeof(int), cudaMemcpyHostToDevice, ops_.stream()), "cudaMemcpyAsync");
        ring_.sent(ops_.stream());
        last_upload_bytes = ints * sizeof(int);

        StepContext ctx;
        ctx.rows = rows;
        ctx.n_seqs = (int)nseq;
        ctx.slots = slots;
        ctx.q_lens = q_lens;
        ctx.max_q_len = *std::max_element(q_lens.begin(), q_lens.end());
        for (size_t k = 0; k < nseq; ++k) ctx.kv_lens.push_back(start[k] + q_lens[k]);
        ctx.max_kv_len = *std::max_element(ctx.kv_lens.begin(), ctx.kv_lens.end());
        ctx.decode = ctx.max_q_len == 1;
        ctx.tokens = dev + offs[0];
        ctx.row_seq = dev + offs[1];
        ctx.row_pos = dev + offs[2];
        ctx.seq_start = dev + offs[4];
        ctx.seq_qlen = dev + offs[5];
        ctx.seq_pos0 = dev + offs[6];
        std::vector<const int*> tables;
        for (size_t g = 0; g < n_groups; ++g) tables.push_back(dev + offs[8 + g]);
        std::vector<CacheView> views;
        for (const auto& call : model_.spec.program)
            views.push_back(call.cache < 0 ? CacheView() : cache_.view(call.cache, call.write, tables, dev + offs[7]));

        DecoderModel::RunOut r = model_.run(ops_, ctx, views, false, layer_arenas);
        if (nwant) {
            Tensor lg = model_.logits(ops_, r.x, dev + offs[3], (int64_t)nwant, nullptr);
            // rows of this pass to their places in the result (consecutive places are copied together)
            size_t w = 0;
            while (w < nwant) {
                size_t e = w + 1;
                while (e < nwant && want_dest[e] == want_dest[e - 1] + 1) ++e;
                cuda_check(cudaMemcpyAsync((float*)result.data + want_dest[w] * vocab, (float*)lg.data + w * vocab,
                                           (e - w) * vocab * sizeof(float), cudaMemcpyDeviceToDevice, ops_.stream()),
                           "cudaMemcpyAsync");
                w = e;
            }
        }
        cache_.commit(slots, q_lens);
        for (size_t k = 0; k < nseq; ++k) done[live[k]] += q_lens[k];
    }
    ops_.arena = nullptr;
    last_logits = result;
    last_queue_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t_begin).count();
    if (total_want && out) {
        cuda_check(cudaMemcpyAsync(out, result.data, total_want * vocab * sizeof(float),
                                   out_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, ops_.stream()),
                   "cudaMemcpyAsync");
    }
    if (out || !total_want) cuda_check(cudaStreamSynchronize(ops_.stream()), "cudaStreamSynchronize");
    return total_want;
}

// ------------------------------------------------------------------ Engine
Engine::Impl::~Impl() {
    kept.clear();
    stepper.reset();
    cache.reset();
    model.reset();
    ops.reset();
    if (stream) cudaStreamDestroy(stream);
}

Engine::Engine(const EngineOptions& opt) : impl_(new Impl) {
    Impl& e = *impl_;
    e.options = opt;
    e.dtype = parse_dtype(opt.dtype);
    if (opt.model_path.empty() == opt.config_json.empty())
        throw Error(ErrorKind::Other, "give either model_path (a model folder) or config_json (random weights)");
    Json cfg;
    if (!opt.model_path.empty()) cfg = read_config_file(opt.model_path);
    else {
        try {
            cfg = Json::parse(opt.config_json);
        } catch (const std::invalid_argument& x) {
            throw ConfigError(std::string("config_json: not JSON: ") + x.what());
        }
    }
    const Architecture arch = friday::architecture(architecture_name_of(cfg));
    e.arch_name = arch.name;
    e.typed_config = arch.read_config(cfg);
    ModelSpec spec = arch.build_spec(e.typed_config);
    e.model.reset(new DecoderModel(spec, e.dtype));
    // weights are checked against the folder before the device is touched: a wrong folder fails fast
    std::unique_ptr<WeightSource> source;
    if (!opt.model_path.empty()) {
        source = open_model_weights(opt.model_path);
        std::vector<Part::Named> all = e.model->named_params(), named;
        std::set<std::string> seen;
        for (auto& p : all)
            if (seen.insert(p.name).second) named.push_back(p);
        check_names(named, *source, spec.ignorable);
    }
    int count = 0;
    cudaError_t err = cudaGetDeviceCount(&count);
    if (err != cudaSuccess || count <= opt.device)
        throw KernelError(format("no CUDA device %d (%s): this library runs on CUDA devices only, it has no CPU path",
                                 opt.device, err != cudaSuccess ? cudaGetErrorString(err) : "not that many devices"));
    e.device = opt.device;
    cuda_check(cudaSetDevice(e.device), "cudaSetDevice");
    cuda_check(cudaStreamCreateWithFlags(&e.stream, cudaStreamNonBlocking), "cudaStreamCreate");
    e.ops.reset(new Ops(e.device, e.stream));
    if (opt.profile) e.ops->set_profile(true);
    if (!source) source = random_weights(e.model->named_params(), opt.seed, "BF16", opt.random_on_device);
    e.model->load(*source, *e.ops);
    source.reset();
    e.max_ctx = (int)std::min<int64_t>(opt.max_ctx, spec.max_positions);
    e.max_batch = opt.max_batch;
    if (e.max_ctx <= 0 || e.max_batch <= 0) throw Error(ErrorKind::Other, "max_ctx and max_batch must be positive");
    const int64_t per_seq = (int64_t)(e.max_ctx + PAGE - 1) / PAGE * PAGE;
    const int64_t max_tokens = opt.max_tokens > 0 ? opt.max_tokens : (int64_t)e.max_batch * per_seq;
    e.cache.reset(new Cache(e.model->cache_requests(), max_tokens, e.max_ctx, e.dtype, e.max_batch, true, e.stream));
    e.stepper.reset(new Stepper(*e.model, *e.cache, *e.ops, opt.prefill_chunk));
}

Engine::~Engine() {}

int Engine::vocabSize() const { return (int)impl_->model->spec.vocab_size; }
int Engine::maxContext() const { return impl_->max_ctx; }
int Engine::maxBatch() const { return impl_->max_batch; }
const Json& Engine::config() const { return impl_->typed_config; }
std::string Engine::architecture() const { return impl_->model->spec.architecture; }
size_t Engine::parameterBytes() const { return impl_->model->parameter_bytes(); }
size_t Engine::cacheBytes() const { return impl_->cache->bytes(); }
void* Engine::stream() const { return (void*)impl_->stream; }
long long Engine::launches() const { return impl_->ops->launches(); }
int* Engine::statusWord() const { return impl_->ops->status_word(); }
int64_t Engine::cacheHeldTokens() const { return impl_->cache->held_tokens(); }
int Engine::cacheHeldSlots() const { return impl_->cache->slots.held_count(); }
int Engine::cacheGroups() const { return (int)impl_->cache->groups.size(); }
int Engine::cacheHeldPages(int g) const { return impl_->cache->groups.at((size_t)g)->pages.held_count(); }

std::string Engine::cacheLayout() const {
    Json out = Json::object(), groups = Json::array(), states = Json::array();
    for (const auto& g : impl_->cache->groups) {
        Json j = Json::object(), ents = Json::array();
        for (int x : g->entries) ents.push(Json(x));
        j.set("entries", ents);
        j.set("window", Json(g->window));
        j.set("pages", Json(g->n_pages));
        j.set("table_width", Json(g->width));
        j.set("n_kv_heads", Json(g->request.n_kv_heads));
        j.set("head_dim", Json(g->request.head_dim));
        groups.push(j);
    }
    for (const auto& kv : impl_->cache->states) states.push(Json(kv.first));
    out.set("groups", groups);
    out.set("states", states);
    return out.dump();
}

std::string Engine::summary() const {
    const Impl& e = *impl_;
    const ModelSpec& s = e.model->spec;
    return format("%s on cuda:%d, %s: %zu layers, width %lld, vocabulary %lld; weights %.2f GB; cache %.2f GB for %lld tokens, "
                  "%d sequences of up to %d",
                  s.architecture.c_str(), e.device, dtype_name(e.dtype), s.layers.size(), (long long)s.width,
                  (long long)s.vocab_size, e.model->parameter_bytes() / 1e9, e.cache->bytes() / 1e9,
                  (long long)e.cache->capacity_tokens(), e.max_batch, e.max_ctx);
}

int Engine::allocSlot() { return impl_->cache->alloc_slot(); }
void Engine::freeSlot(int slot) { impl_->cache->free_slot(slot); }
int Engine::slotLength(int slot) const {
    if (!impl_->cache->slots.holds(slot)) throw CacheError(format("slot %d is not held", slot));
    return impl_->cache->lens[slot];
}

size_t Engine::step(const StepBatch& batch, float* logits, bool on_device) {
    Impl& e = *impl_;
    cuda_check(cudaSetDevice(e.device), "cudaSetDevice");
    if (!e.options.profile) return e.stepper->step(batch, logits, on_device);
    const auto t0 = std::chrono::steady_clock::now();
    const size_t rows = e.stepper->step(batch, logits, on_device);
    e.prof.host_ms += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    e.prof.steps += 1;
    return rows;
}

static int single_at(Engine::Impl& e, int pos) {
    if (pos == 0) {
        if (e.single >= 0) e.cache->free_slot(e.single);
        e.single = -1;
        e.single = e.cache->alloc_slot();
    }
    const int have = e.single < 0 ? 0 : e.cache->lens[e.single];
    if (e.single < 0 || have != pos)
        throw StepError(format("positions must be fed in order, starting at 0 for a new sequence (at %d, got %d)", have, pos));
    return e.single;
}

void Engine::step(int token, int pos, float* logits) {
    StepBatch b;
    b.slots = {single_at(*impl_, pos)};
    b.tokens = {{token}};
    b.want = {{0}};
    step(b, logits, false);
    check();
}

void Engine::prefill(const int* tokens, int n, int pos, float* logits) {
    if (n <= 0) throw StepError("prefill needs at least one token");
    StepBatch b;
    b.slots = {single_at(*impl_, pos)};
    b.tokens = {std::vector<int>(tokens, tokens + n)};
    b.want = {{n - 1}};
    step(b, logits, false);
    check();
}

void Engine::check() { impl_->ops->check_status(); }

Profile Engine::profile() {
    Impl& e = *impl_;
    double ms[Ops::Segments];
    long long calls[Ops::Segments];
    e.ops->take_profile(ms, calls);
    Profile p = e.prof;
    p.product_ms = ms[Ops::Product];
    p.attention_ms = ms[Ops::Attention];
    p.other_ms = ms[Ops::Other];
    p.product_calls = calls[Ops::Product];
    p.attention_calls = calls[Ops::Attention];
    p.other_calls = calls[Ops::Other];
    e.prof = Profile();
    return p;
}

std::unique_ptr<Decoder> Engine::decoder(const std::vector<int>& slots, const std::vector<int>& first_tokens,
                                         float temperature, uint64_t seed, const std::vector<int>& streams,
                                         const std::vector<int>& steps_done) {
    Impl& e = *impl_;
    cuda_check(cudaSetDevice(e.device), "cudaSetDevice");
    auto it = e.kept.find((int)slots.size());
    if (it != e.kept.end()) {
        std::unique_ptr<Decoder> d = std::move(it->second);
        e.kept.erase(it);
        if (reset_device_decoder(*d, slots, first_tokens, temperature, seed, streams, steps_done)) return d;
    }
    return make_device_decoder(e, slots, first_tokens, temperature, seed, streams, steps_done);
}

void Engine::keepDecoder(std::unique_ptr<Decoder> d) {
    if (d) impl_->kept[d->rows()] = std::move(d);
}

std::vector<Generation> Engine::generate(const std::vector<std::vector<int>>& prompts, const GenerateOptions& opt) {
    Impl& e = *impl_;
    if (opt.temperature < 0) throw GenerationError("temperature must not be negative");
    cuda_check(cudaSetDevice(e.device), "cudaSetDevice");
    SamplingParams sp;
    sp.temperature = opt.temperature;
    sp.seed = opt.seed;
    Sampler sampler(*e.ops, sp);
    std::unique_ptr<Decoder> dec;
    LoopHooks hooks;
    hooks.alloc_slot = [&]() { return allocSlot(); };
    hooks.free_slot = [&](int s) { freeSlot(s); };
    hooks.step = [&](const std::vector<int>& slots, const std::vector<std::vector<int>>& toks,
                     const std::vector<std::vector<int>>& want) {
        StepBatch b;
        b.slots = slots;
        b.tokens = toks;
        b.want = want;
        step(b, nullptr, false);                       // the logits stay on the device for the sampler
    };
    hooks.sample = [&](const std::vector<int>& streams, const std::vector<int>& steps) {
        return sampler.sample(e.stepper->last_logits, streams, steps);
    };
    hooks.decoder = [&](const std::vector<int>& slots, const std::vector<int>& firsts, const std::vector<int>& streams,
                        const std::vector<int>& done) {
        dec = decoder(slots, firsts, opt.temperature, opt.seed, streams, done);
        LoopHooks::Rows rows;
        rows.step = [&](const std::vector<int>& tokens) {
            dec->step(tokens.data());
            return dec->sampled();
        };
        rows.retire = [&](int row) { dec->retire(row); };
        rows.close = [&]() { keepDecoder(std::move(dec)); };
        return rows;
    };
    std::vector<Generation> out = generate_loop(prompts, hooks, e.max_batch, e.max_ctx, vocabSize(), opt);
    check();
    return out;
}

}  // namespace friday
