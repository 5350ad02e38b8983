// The C interface (capi.h): every function catches what the library throws and turns it into an error kind and a
// message that the caller reads afterwards.
#include "friday/capi.h"

#include <string.h>

#include <algorithm>
#include <set>

#include "engine/engine_impl.h"
#include "friday/weights.h"
#include "ops/kernels.h"

using namespace friday;

#define FR_API extern "C" __attribute__((visibility("default")))

namespace {
thread_local std::string g_error, g_detail, g_text;

int fail(const std::exception& x) {
    g_error = x.what();
    g_detail.clear();
    int kind = 0;
    if (const Error* e = dynamic_cast<const Error*>(&x)) kind = (int)e->kind;
    if (const WeightsError* w = dynamic_cast<const WeightsError*>(&x)) {
        Json d = Json::object(), miss = Json::array(), unexp = Json::array(), wrong = Json::array();
        for (const auto& n : w->missing) miss.push(Json(n));
        for (const auto& n : w->unexpected) unexp.push(Json(n));
        for (const auto& s : w->wrong_shape) {
            Json e = Json::array(), got = Json::array(), want = Json::array();
            for (int64_t v : s.got) got.push(Json(v));
            for (int64_t v : s.want) want.push(Json(v));
            e.push(Json(s.name));
            e.push(got);
            e.push(want);
            wrong.push(e);
        }
        d.set("missing", miss);
        d.set("unexpected", unexp);
        d.set("wrong_shape", wrong);
        g_detail = d.dump();
    }
    return 100 + kind;
}

#define GUARD(...)                                   \
    try {                                            \
        __VA_ARGS__;                                 \
        return 0;                                    \
    } catch (const std::exception& x) {              \
        return fail(x);                              \
    }

const char* hand_back(const std::string& s) {
    g_text = s;
    return g_text.c_str();
}

Json parse_arg(const char* text, const char* what) {
    try {
        return Json::parse(text ? text : "null");
    } catch (const std::invalid_argument& x) {
        throw Error(ErrorKind::Other, std::string(what) + ": not JSON: " + x.what());
    }
}

Json ints_json(const std::vector<int64_t>& v) {
    Json a = Json::array();
    for (int64_t x : v) a.push(Json(x));
    return a;
}
Json ints_json(const std::vector<int>& v) {
    Json a = Json::array();
    for (int x : v) a.push(Json(x));
    return a;
}

Json request_json(const CacheRequest& r) {
    Json j = Json::object();
    j.set("kind", Json(r.kind == CacheRequest::KV ? "kv" : r.kind == CacheRequest::State ? "state" : "none"));
    if (r.kind == CacheRequest::KV) {
        j.set("n_kv_heads", Json(r.n_kv_heads));
        j.set("head_dim", Json(r.head_dim));
        j.set("window", Json(r.window));
    } else if (r.kind == CacheRequest::State) {
        j.set("shape", ints_json(r.state_shape));
        j.set("dtype", Json(dtype_name(r.state_dtype)));
    }
    return j;
}

CacheRequest request_from(const Json& j) {
    const std::string kind = j.get_string("kind", "none");
    if (kind == "kv") return CacheRequest::kv((int)j.get_int("n_kv_heads", 0), (int)j.get_int("head_dim", 0), (int)j.get_int("window", 0));
    if (kind == "state") {
        std::vector<int64_t> shape;
        if (const Json* s = j.find("shape"))
            for (const Json& d : s->items()) shape.push_back(d.as_int());
        return CacheRequest::state(shape, parse_dtype(j.get_string("dtype", "float32")));
    }
    if (kind == "none") return CacheRequest();
    throw CacheError("a cache entry asks for '" + kind + "', which is neither keys and values nor a state");
}

std::vector<std::vector<int>> ragged(int n, const int* offsets, const int* values) {
    std::vector<std::vector<int>> out((size_t)n);
    for (int i = 0; i < n; ++i) out[i].assign(values + offsets[i], values + offsets[i + 1]);
    return out;
}

GenerateOptions generate_options(const Json& j) {
    GenerateOptions o;
    o.max_new_tokens = (int)j.get_int("max_new_tokens", o.max_new_tokens);
    o.temperature = (float)j.get_double("temperature", 0.0);
    o.seed = (uint64_t)j.get_int("seed", 0);
    o.ignore_eos = j.get_bool("ignore_eos", false);
    if (const Json* s = j.find("stop_token_ids"))
        for (const Json& t : s->items()) o.stop_token_ids.push_back((int)t.as_int());
    return o;
}

Json generations_json(const std::vector<Generation>& gens) {
    Json out = Json::array();
    for (const auto& g : gens) {
        Json j = Json::object();
        j.set("tokens", ints_json(g.tokens));
        j.set("finish_reason", Json(g.finish_reason));
        out.push(j);
    }
    return out;
}

struct HookFailure : std::runtime_error {
    int code;
    explicit HookFailure(int c) : std::runtime_error("a callback of the generation loop failed"), code(c) {}
};

inline const Tensor* T(const FridayTensor* t) { return (const Tensor*)t; }
inline Tensor* T(FridayTensor* t) { return (Tensor*)t; }

CacheView view_of(const FridayKV* kv) {
    CacheView v;
    if (!kv) return v;
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
    return v;
}

struct OpsHandle {
    std::unique_ptr<Ops> ops;
    std::unique_ptr<Arena> arena;
    Ops& begin() {
        cuda_check(cudaSetDevice(ops->device()), "cudaSetDevice");
        arena->reset();
        ops->arena = arena.get();
        return *ops;
    }
    void copy_out(const Tensor& src, FridayTensor* dst) {
        Tensor& d = *T(dst);
        if (d.rows() != src.rows() || d.cols() != src.cols() || d.dtype != src.dtype)
            throw KernelError("the tensor given for a result has another shape or dtype than the result");
        const size_t es = dtype_size(src.dtype);
        cuda_check(cudaMemcpy2DAsync(d.data, (size_t)d.ld * es, src.data, (size_t)src.ld * es, (size_t)src.cols() * es,
                                     (size_t)src.rows(), cudaMemcpyDeviceToDevice, ops->stream()), "cudaMemcpy2DAsync");
    }
};

Rows rows_of(const FridayTensor* x, const FridayTensor* ssq, float eps, const FridayTensor* source = nullptr,
             const FridayTensor* norm_weight = nullptr) {
    Rows r(*T(x));
    if (ssq && ssq->data) {
        r.deferred = true;
        r.ssq = *T(ssq);
        r.eps = eps;
        if (source) r.source = *T(source);
        if (norm_weight) r.weight = *T(norm_weight);
    }
    return r;
}

static_assert(sizeof(FridayTensor) == sizeof(Tensor), "FridayTensor must mirror friday::Tensor");

}  // namespace

FR_API const char* friday_last_error(void) { return g_error.c_str(); }
FR_API const char* friday_last_error_detail(void) { return g_detail.c_str(); }
FR_API int friday_set_builder(int (*build)(const char*)) { GUARD(kernels::set_builder(build)) }
FR_API int friday_load_plugin(const char* path) { GUARD(load_plugin(path)) }
FR_API const char* friday_loaded_libraries(void) { return hand_back(kernels::loaded_libraries()); }

// ------------------------------------------------------------------ configuration
FR_API int friday_read_config(const char* config_json, const char** typed_json) {
    GUARD({
        const Json cfg = parse_arg(config_json, "config.json");
        const Architecture arch = architecture(architecture_name_of(cfg));
        *typed_json = hand_back(arch.read_config(cfg).dump());
    })
}

FR_API int friday_registered(const char* what, const char** json_list) {
    GUARD({
        Json a = Json::array();
        const std::string w = what;
        for (const auto& n : (w == "architectures" ? registered_architectures() : registered_parts(w))) a.push(Json(n));
        *json_list = hand_back(a.dump());
    })
}

FR_API int friday_describe_model(const char* config_json, const char** json) {
    GUARD({
        const Json cfg = parse_arg(config_json, "config.json");
        const Architecture arch = architecture(architecture_name_of(cfg));
        const Json typed = arch.read_config(cfg);
        ModelSpec spec = arch.build_spec(typed);
        DecoderModel model(spec, DType::BF16);
        Json out = Json::object();
        out.set("architecture", Json(spec.architecture));
        out.set("config", typed);
        out.set("vocab_size", Json(spec.vocab_size));
        out.set("width", Json(spec.width));
        out.set("max_positions", Json(spec.max_positions));
        out.set("n_layers", Json((int64_t)spec.layers.size()));
        Json program = Json::array();
        for (const auto& c : spec.program) {
            Json e = Json::object();
            e.set("layer", Json(c.layer));
            e.set("cache", Json(c.cache));
            e.set("write", Json(c.write));
            program.push(e);
        }
        out.set("program", program);
        Json reqs = Json::object();
        for (const auto& kv : model.cache_requests()) reqs.set(std::to_string(kv.first), request_json(kv.second));
        out.set("cache_requests", reqs);
        Json params = Json::array();
        std::set<std::string> seen;
        for (const auto& p : model.named_params()) {
            if (!seen.insert(p.name).second) continue;
            Json e = Json::object();
            e.set("name", Json(p.name));
            e.set("shape", ints_json(p.decl.shape));
            e.set("integer", Json(p.decl.integer));
            e.set("one", Json(p.decl.one));
            params.push(e);
        }
        out.set("params", params);
        Json ign = Json::array();
        for (const auto& n : spec.ignorable) ign.push(Json(n));
        out.set("ignorable", ign);
        *json = hand_back(out.dump());
    })
}

// ------------------------------------------------------------------ weights
FR_API int friday_write_random_model(const char* dir, const char* config_json, uint64_t seed, const char* dtype, int shards) {
    GUARD(write_random_model(dir, parse_arg(config_json, "config.json"), seed, dtype ? dtype : "BF16", shards))
}

FR_API int friday_check_weights(const char* model_dir) {
    GUARD({
        const Json cfg = read_config_file(model_dir);
        const Architecture arch = architecture(architecture_name_of(cfg));
        ModelSpec spec = arch.build_spec(arch.read_config(cfg));
        DecoderModel model(spec, DType::BF16);
        std::unique_ptr<WeightSource> src = open_model_weights(model_dir);
        std::vector<Part::Named> named;
        std::set<std::string> seen;
        for (auto& p : model.named_params())
            if (seen.insert(p.name).second) named.push_back(p);
        check_names(named, *src, spec.ignorable);
    })
}

FR_API int friday_storage_plan(const char* model_dir, const char* dtype, const char** json) {
    GUARD({
        const Json cfg = read_config_file(model_dir);
        const Architecture arch = architecture(architecture_name_of(cfg));
        DecoderModel model(arch.build_spec(arch.read_config(cfg)), parse_dtype(dtype));
        std::unique_ptr<WeightSource> src = open_model_weights(model_dir);
        Json out = Json::array();
        for (const auto& s : model.plan_storage(*src)) {
            Json e = Json::object();
            e.set("name", Json(s.param.name));
            e.set("dtype", Json(dtype_name(s.dtype)));
            e.set("into", Json(s.param.decl.into));
            out.push(e);
        }
        *json = hand_back(out.dump());
    })
}

FR_API int friday_random_tensor(uint64_t seed, const char* name, int one, int64_t count, float* out) {
    GUARD(random_tensor_host(seed, name, one != 0, count, out))
}

namespace {
struct StHandle {
    std::unique_ptr<SafetensorsFile> file;          // a single file, or
    std::string dir;                                // a folder: names come from the source, bytes from the files
    std::vector<std::unique_ptr<SafetensorsFile>> shards;
};
}  // namespace

FR_API int friday_safetensors_open(const char* path, void** handle) {
    GUARD({
        auto h = std::make_unique<StHandle>();
        h->file.reset(new SafetensorsFile(path));
        *handle = h.release();
    })
}

FR_API int friday_safetensors_list(void* handle, const char** json) {
    GUARD({
        StHandle* h = (StHandle*)handle;
        Json out = Json::object(), tensors = Json::array();
        for (const auto& n : h->file->names()) {
            StoredTensor t;
            h->file->info(n, &t);
            Json e = Json::object();
            e.set("name", Json(n));
            e.set("dtype", Json(t.dtype));
            e.set("shape", ints_json(t.shape));
            tensors.push(e);
        }
        out.set("tensors", tensors);
        out.set("metadata", h->file->metadata());
        *json = hand_back(out.dump());
    })
}

FR_API int friday_safetensors_read(void* handle, const char* name, void* out, size_t bytes) {
    GUARD({
        StHandle* h = (StHandle*)handle;
        size_t n = 0;
        const void* p = h->file->bytes(name, &n);
        if (!p) throw WeightsError(h->file->path() + ": no tensor '" + name + "'");
        if (n != bytes) throw WeightsError(format("tensor '%s' has %zu bytes, the caller expects %zu", name, n, bytes));
        memcpy(out, p, n);
    })
}

FR_API void friday_safetensors_free(void* handle) { delete (StHandle*)handle; }

FR_API int friday_safetensors_write(const char* path, const char* header_json, const void* const* blobs, const char* metadata_json) {
    GUARD({
        const Json header = parse_arg(header_json, "header");
        std::vector<HostTensor> tensors;
        for (size_t i = 0; i < header.size(); ++i) {
            const Json& e = header[i];
            HostTensor t;
            t.name = e.at("name").as_string();
            t.dtype = e.at("dtype").as_string();
            for (const Json& d : e.at("shape").items()) t.shape.push_back(d.as_int());
            int64_t n = 1;
            for (int64_t d : t.shape) n *= d;
            const size_t bytes = (size_t)n * stored_dtype_size(t.dtype);
            t.bytes.assign((const uint8_t*)blobs[i], (const uint8_t*)blobs[i] + bytes);
            tensors.push_back(std::move(t));
        }
        write_safetensors(path, tensors, metadata_json ? parse_arg(metadata_json, "metadata") : Json());
    })
}

// ------------------------------------------------------------------ the cache's book-keeping
FR_API int friday_cache_new(const char* requests_json, int64_t max_tokens, int max_seq_tokens, int max_slots, void** handle) {
    GUARD({
        const Json j = parse_arg(requests_json, "requests");
        std::map<int, CacheRequest> reqs;
        for (const auto& m : j.members()) reqs[atoi(m.first.c_str())] = request_from(m.second);
        *handle = new Cache(reqs, max_tokens, max_seq_tokens, DType::F32, max_slots, false);
    })
}
FR_API void friday_cache_free(void* c) { delete (Cache*)c; }
FR_API int friday_cache_alloc_slot(void* c, int* slot) { GUARD(*slot = ((Cache*)c)->alloc_slot()) }
FR_API int friday_cache_free_slot(void* c, int slot) { GUARD(((Cache*)c)->free_slot(slot)) }
FR_API int friday_cache_reserve(void* c, int n, const int* slots, const int* q) {
    GUARD(((Cache*)c)->reserve(std::vector<int>(slots, slots + n), std::vector<int>(q, q + n)))
}
FR_API int friday_cache_commit(void* c, int n, const int* slots, const int* q) {
    GUARD(((Cache*)c)->commit(std::vector<int>(slots, slots + n), std::vector<int>(q, q + n)))
}

static Json cache_json(const Cache& c) {
    Json out = Json::object(), groups = Json::array(), states = Json::object();
    out.set("max_slots", Json(c.max_slots));
    out.set("slots_held", Json(c.slots.held_count()));
    out.set("slots_free", Json(c.slots.free_count()));
    out.set("lens", ints_json(c.lens));
    Json held = Json::array();
    for (int s = 0; s < c.max_slots; ++s) held.push(Json(c.slots.holds(s)));
    out.set("held", held);
    for (const auto& g : c.groups) {
        Json j = Json::object();
        j.set("entries", ints_json(g->entries));
        j.set("window", Json(g->window));
        j.set("n_pages", Json(g->n_pages));
        j.set("width", Json(g->width));
        j.set("pages_held", Json(g->pages.held_count()));
        j.set("pages_free", Json(g->pages.free_count()));
        j.set("pool_shape", ints_json(std::vector<int64_t>{(int64_t)g->entries.size(), g->n_pages, PAGE, g->request.n_kv_heads,
                                                            g->request.head_dim}));
        Json table = Json::array();
        for (int s = 0; s < c.max_slots; ++s) table.push(ints_json(std::vector<int>(g->table_row(s), g->table_row(s) + g->width)));
        j.set("table", table);
        groups.push(j);
    }
    out.set("groups", groups);
    for (const auto& kv : c.states) {
        std::vector<int64_t> shape{(int64_t)c.max_slots};
        shape.insert(shape.end(), kv.second.shape.begin(), kv.second.shape.end());
        states.set(std::to_string(kv.first), ints_json(shape));
    }
    out.set("states", states);
    Json group_of = Json::object();
    for (const auto& kv : c.group_of) group_of.set(std::to_string(kv.first), Json(kv.second));
    out.set("group_of", group_of);
    return out;
}

FR_API int friday_cache_info(void* c, const char** json) { GUARD(*json = hand_back(cache_json(*(Cache*)c).dump())) }

// ------------------------------------------------------------------ the generation loop alone
FR_API int friday_generate_loop(int n_prompts, const int* offsets, const int* tokens, const FridayLoopHooks* h, int max_batch,
                                int max_context, int vocab_size, const char* options_json, const char** result_json) {
    GUARD({
        LoopHooks hooks;
        auto flat = [](const std::vector<std::vector<int>>& v, std::vector<int>& off, std::vector<int>& val) {
            off.assign(1, 0);
            val.clear();
            for (const auto& x : v) {
                val.insert(val.end(), x.begin(), x.end());
                off.push_back((int)val.size());
            }
        };
        hooks.step = [&](const std::vector<int>& slots, const std::vector<std::vector<int>>& toks,
                         const std::vector<std::vector<int>>& want) {
            std::vector<int> to, tv, wo, wv;
            flat(toks, to, tv);
            flat(want, wo, wv);
            const int rc = h->step(h->user, (int)slots.size(), slots.data(), to.data(), tv.data(), wo.data(), wv.data());
            if (rc) throw HookFailure(rc);
        };
        hooks.sample = [&](const std::vector<int>& streams, const std::vector<int>& steps) {
            std::vector<int> out(streams.size());
            const int rc = h->sample(h->user, (int)streams.size(), streams.data(), steps.data(), out.data());
            if (rc) throw HookFailure(rc);
            return out;
        };
        hooks.alloc_slot = [&]() {
            int s = -1;
            const int rc = h->alloc_slot(h->user, &s);
            if (rc) throw HookFailure(rc);
            return s;
        };
        hooks.free_slot = [&](int s) {
            const int rc = h->free_slot(h->user, s);
            if (rc) throw HookFailure(rc);
        };
        const GenerateOptions opt = generate_options(parse_arg(options_json, "options"));
        *result_json = hand_back(generations_json(generate_loop(ragged(n_prompts, offsets, tokens), hooks, max_batch,
                                                                max_context, vocab_size, opt)).dump());
    })
}

// ------------------------------------------------------------------ the engine
FR_API int friday_engine_new(const char* options_json, void** engine) {
    GUARD({
        const Json j = parse_arg(options_json, "options");
        EngineOptions o;
        o.model_path = j.get_string("model_path", "");
        if (const Json* c = j.find("config")) {
            if (c->is_object()) o.config_json = c->dump();
            else if (c->is_string()) o.config_json = c->as_string();
        }
        o.seed = (uint64_t)j.get_int("seed", 0);
        o.dtype = j.get_string("dtype", o.dtype);
        o.max_ctx = (int)j.get_int("max_ctx", o.max_ctx);
        o.max_batch = (int)j.get_int("max_batch", o.max_batch);
        o.max_tokens = j.get_int("max_tokens", 0);
        o.device = (int)j.get_int("device", 0);
        o.prefill_chunk = (int)j.get_int("prefill_chunk", o.prefill_chunk);
        o.cuda_graphs = j.get_bool("cuda_graphs", true);
        o.random_on_device = j.get_bool("random_on_device", true);
        o.profile = j.get_bool("profile", false);
        *engine = new Engine(o);
    })
}
FR_API void friday_engine_free(void* e) { delete (Engine*)e; }

FR_API int friday_engine_info(void* e, const char** json) {
    GUARD({
        Engine& eng = *(Engine*)e;
        Json j = Json::object();
        j.set("vocab_size", Json(eng.vocabSize()));
        j.set("max_context", Json(eng.maxContext()));
        j.set("max_batch", Json(eng.maxBatch()));
        j.set("summary", Json(eng.summary()));
        j.set("architecture", Json(eng.architecture()));
        j.set("config", eng.config());
        j.set("parameter_bytes", Json((int64_t)eng.parameterBytes()));
        j.set("cache_bytes", Json((int64_t)eng.cacheBytes()));
        j.set("stream", Json((int64_t)(intptr_t)eng.stream()));
        j.set("status_word", Json((int64_t)(intptr_t)eng.statusWord()));
        j.set("n_layers", Json((int64_t)eng.impl()->model->spec.layers.size()));
        j.set("width", Json(eng.impl()->model->spec.width));
        j.set("device", Json(eng.impl()->device));
        j.set("dtype", Json(dtype_name(eng.impl()->dtype)));
        j.set("sm_count", Json(eng.impl()->ops->sm_count()));
        *json = hand_back(j.dump());
    })
}

FR_API int friday_engine_alloc_slot(void* e, int* slot) { GUARD(*slot = ((Engine*)e)->allocSlot()) }
FR_API int friday_engine_free_slot(void* e, int slot) { GUARD(((Engine*)e)->freeSlot(slot)) }
FR_API int friday_engine_slot_length(void* e, int slot, int* length) { GUARD(*length = ((Engine*)e)->slotLength(slot)) }

FR_API int friday_engine_step(void* e, int n, const int* slots, const int* token_offsets, const int* tokens,
                              const int* want_offsets, const int* want, float* logits, int on_device, int64_t* rows) {
    GUARD({
        StepBatch b;
        b.slots.assign(slots, slots + n);
        b.tokens = ragged(n, token_offsets, tokens);
        b.want = ragged(n, want_offsets, want);
        const size_t r = ((Engine*)e)->step(b, logits, on_device != 0);
        if (rows) *rows = (int64_t)r;
    })
}
FR_API int friday_engine_step_token(void* e, int token, int pos, float* logits) { GUARD(((Engine*)e)->step(token, pos, logits)) }
FR_API int friday_engine_prefill(void* e, const int* tokens, int n, int pos, float* logits) {
    GUARD(((Engine*)e)->prefill(tokens, n, pos, logits))
}

FR_API int friday_engine_generate(void* e, int n_prompts, const int* offsets, const int* tokens, const char* options_json,
                                  friday_on_step on_step, void* user, const char** result_json) {
    GUARD({
        GenerateOptions opt = generate_options(parse_arg(options_json, "options"));
        if (on_step)
            opt.on_step = [=](const std::vector<int>& reqs, const std::vector<int>& toks) {
                on_step(user, (int)reqs.size(), reqs.data(), toks.data());
            };
        *result_json = hand_back(generations_json(((Engine*)e)->generate(ragged(n_prompts, offsets, tokens), opt)).dump());
    })
}

FR_API int friday_engine_set_trace(void* e, void* trace, int launches) {
    GUARD(((Engine*)e)->impl()->ops->set_trace((unsigned long long*)trace, launches))
}

FR_API int friday_engine_check(void* e) { GUARD(((Engine*)e)->check()) }

FR_API int friday_engine_profile(void* e, const char** json) {
    GUARD({
        const Profile p = ((Engine*)e)->profile();
        Json j = Json::object();
        j.set("steps", Json((int64_t)p.steps));
        j.set("host_ms", Json(p.host_ms));
        j.set("product_ms", Json(p.product_ms));
        j.set("attention_ms", Json(p.attention_ms));
        j.set("other_ms", Json(p.other_ms));
        j.set("product_calls", Json((int64_t)p.product_calls));
        j.set("attention_calls", Json((int64_t)p.attention_calls));
        j.set("other_calls", Json((int64_t)p.other_calls));
        *json = hand_back(j.dump());
    })
}

FR_API int friday_engine_stats(void* e, const char** json) {
    GUARD({
        Engine& eng = *(Engine*)e;
        Json j = cache_json(*eng.impl()->cache);
        j.set("launches", Json((int64_t)eng.launches()));
        j.set("held_tokens", Json(eng.cacheHeldTokens()));
        j.set("last_upload_bytes", Json((int64_t)eng.impl()->stepper->last_upload_bytes));
        j.set("last_queue_ms", Json(eng.impl()->stepper->last_queue_ms));
        j.set("kept_decoders", Json((int64_t)eng.impl()->kept.size()));
        *json = hand_back(j.dump());
    })
}

// ------------------------------------------------------------------ decoders
FR_API int friday_decoder_new(void* e, int n, const int* slots, const int* firsts, float temperature, uint64_t seed,
                              const int* streams, const int* steps_done, void** decoder) {
    GUARD({
        std::vector<int> st, sd;
        if (streams) st.assign(streams, streams + n);
        if (steps_done) sd.assign(steps_done, steps_done + n);
        *decoder = ((Engine*)e)->decoder(std::vector<int>(slots, slots + n), std::vector<int>(firsts, firsts + n), temperature,
                                         seed, st, sd).release();
    })
}
FR_API int friday_decoder_step(void* d, const int* tokens) { GUARD(((Decoder*)d)->step(tokens)) }
FR_API int friday_decoder_sampled(void* d, int* out) {
    GUARD({
        const std::vector<int> s = ((Decoder*)d)->sampled();
        memcpy(out, s.data(), s.size() * sizeof(int));
    })
}
FR_API int friday_decoder_logits(void* d, float* out, int on_device) { GUARD(((Decoder*)d)->logits(out, on_device != 0)) }
FR_API int friday_decoder_retire(void* d, int row) { GUARD(((Decoder*)d)->retire(row)) }
FR_API int friday_decoder_info(void* d, const char** json) {
    GUARD({
        Decoder& dec = *(Decoder*)d;
        Json j = Json::object();
        j.set("rows", Json(dec.rows()));
        j.set("launches_per_step", Json((int64_t)dec.launchesPerStep()));
        j.set("graphs", Json(dec.graphsCaptured()));
        j.set("bound", Json(dec.bound()));
        *json = hand_back(j.dump());
    })
}
FR_API int friday_decoder_close(void* e, void* d) { GUARD(((Engine*)e)->keepDecoder(std::unique_ptr<Decoder>((Decoder*)d))) }
FR_API void friday_decoder_free(void* d) { delete (Decoder*)d; }

// ------------------------------------------------------------------ operations
FR_API int friday_ops_new(int device, void* stream, void** ops) {
    GUARD({
        auto h = std::make_unique<OpsHandle>();
        h->ops.reset(new Ops(device, (cudaStream_t)stream));
        h->arena.reset(new Arena((cudaStream_t)stream));
        *ops = h.release();
    })
}
FR_API void friday_ops_free(void* ops) { delete (OpsHandle*)ops; }

FR_API int friday_ops_embedding(void* h, const int* tokens, int64_t n, const FridayTensor* table, FridayTensor* out) {
    GUARD(((OpsHandle*)h)->begin().embedding(tokens, n, *T(table), T(out)))
}
FR_API int friday_ops_gather_rows(void* h, const int* rows, int64_t n, const FridayTensor* src, FridayTensor* out) {
    GUARD({
        OpsHandle& o = *(OpsHandle*)h;
        o.copy_out(o.begin().gather_rows(rows, n, *T(src)), out);
    })
}
FR_API int friday_ops_rmsnorm(void* h, const FridayTensor* x, const FridayTensor* w, float eps, FridayTensor* out) {
    GUARD(((OpsHandle*)h)->begin().rmsnorm(*T(x), *T(w), eps, T(out)))
}
FR_API int friday_ops_swiglu(void* h, const FridayTensor* gu, FridayTensor* out) {
    GUARD({
        OpsHandle& o = *(OpsHandle*)h;
        o.copy_out(o.begin().swiglu(*T(gu)), out);
    })
}
FR_API int friday_ops_rope_kv_write(void* h, FridayTensor* qkv, const int* row_seq, const int* row_pos, const float* denom,
                                    int rotary_dim, int nq, int nkv, int hd, const FridayKV* kv) {
    GUARD({
        CacheView v = view_of(kv);
        ((OpsHandle*)h)->begin().rope_kv_write(*T(qkv), row_seq, row_pos, denom, rotary_dim, nq, nkv, hd, kv ? &v : nullptr);
    })
}
FR_API int friday_ops_advance(void* h, int* tokens, const int* sampled, int* row_pos, int* kv_len, const int* row_seq,
                              int* draws, int n) {
    GUARD(((OpsHandle*)h)->begin().advance(tokens, sampled, row_pos, kv_len, row_seq, draws, n))
}
FR_API int friday_ops_scale_rows(void* h, FridayTensor* x, float scale) { GUARD(((OpsHandle*)h)->begin().scale_rows(*T(x), scale)) }
FR_API int friday_ops_finish_logits(void* h, FridayTensor* logits, const FridayTensor* bias, float scale, float softcap) {
    GUARD(((OpsHandle*)h)->begin().finish_logits(*T(logits), bias ? T(bias) : nullptr, scale, softcap))
}
FR_API int friday_ops_linear(void* h, const FridayTensor* x, const FridayTensor* ssq, float eps, const FridayTensor* source,
                             const FridayTensor* norm_weight, const FridayTensor* weight, const FridayTensor* bias,
                             const FridayTensor* residual, FridayTensor* out) {
    GUARD(((OpsHandle*)h)->begin().linear(rows_of(x, ssq, eps, source, norm_weight), *T(weight), bias ? T(bias) : nullptr,
                                          residual ? T(residual) : nullptr, out->dtype, T(out)))
}
FR_API int friday_ops_linear_tc(void* h, const FridayTensor* x, const FridayTensor* weight, const FridayTensor* bias,
                                const FridayTensor* residual, FridayTensor* out, int swap, int bn, int splits, int act) {
    GUARD(((OpsHandle*)h)->begin().linear_tc(*T(x), *T(weight), bias ? T(bias) : nullptr, residual ? T(residual) : nullptr,
                                             *T(out), swap, bn, splits, act, nullptr))
}
FR_API int friday_ops_linear_simt(void* h, const FridayTensor* x, const FridayTensor* weight, const FridayTensor* bias,
                                  const FridayTensor* residual, FridayTensor* out) {
    GUARD(((OpsHandle*)h)->begin().linear_simt(*T(x), *T(weight), bias ? T(bias) : nullptr, residual ? T(residual) : nullptr, *T(out)))
}
FR_API int friday_ops_linear_norm(void* h, const FridayTensor* x, const FridayTensor* in_ssq, float in_eps,
                                  const FridayTensor* weight, const FridayTensor* norm_weight, float eps,
                                  const FridayTensor* bias, const FridayTensor* residual, FridayTensor* out,
                                  FridayTensor* normed, FridayTensor* ssq, int* deferred) {
    GUARD({
        OpsHandle& o = *(OpsHandle*)h;
        auto r = o.begin().linear_norm(rows_of(x, in_ssq, in_eps), *T(weight), *T(norm_weight), eps, bias ? T(bias) : nullptr,
                                       residual ? T(residual) : nullptr);
        o.copy_out(r.first, out);
        o.copy_out(r.second.t, normed);
        *deferred = r.second.deferred ? 1 : 0;
        if (r.second.deferred) {
            if (ssq->shape[0] < r.second.ssq.rows() || ssq->shape[1] != r.second.ssq.cols())
                throw KernelError("linear_norm: the tensor given for the partial sums is too small");
            ssq->shape[0] = r.second.ssq.rows();
            o.copy_out(r.second.ssq, ssq);
        }
    })
}
FR_API int friday_ops_qkv_rope_write(void* h, const FridayTensor* x, const FridayTensor* in_ssq, float in_eps,
                                     const FridayTensor* weight, const FridayTensor* bias, const int* row_seq,
                                     const int* row_pos, const float* denom, int rotary_dim, int nq, int nkv, int hd,
                                     const FridayKV* kv, FridayTensor* out) {
    GUARD({
        OpsHandle& o = *(OpsHandle*)h;
        CacheView v = view_of(kv);
        o.copy_out(o.begin().qkv_rope_write(rows_of(x, in_ssq, in_eps), *T(weight), bias ? T(bias) : nullptr, row_seq, row_pos,
                                            denom, rotary_dim, nq, nkv, hd, kv ? &v : nullptr), out);
    })
}
FR_API int friday_ops_linear_swiglu(void* h, const FridayTensor* x, const FridayTensor* in_ssq, float in_eps,
                                    const FridayTensor* weight_pairs, FridayTensor* out) {
    GUARD({
        OpsHandle& o = *(OpsHandle*)h;
        o.copy_out(o.begin().linear_swiglu(rows_of(x, in_ssq, in_eps), *T(weight_pairs)), out);
    })
}
FR_API int friday_ops_attention(void* h, const FridayTensor* q, int64_t q_stride, FridayTensor* out, const FridayKV* kv,
                                const FridayGeometry* g, int nq, int nkv, int hd, int window, float scale) {
    GUARD({
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
        ((OpsHandle*)h)->begin().attention(*T(q), q_stride, *T(out), view_of(kv), ctx, nq, nkv, hd, window, scale);
    })
}
FR_API int friday_ops_sample(void* h, const FridayTensor* logits, const float* temperature, const int* streams,
                             const int* steps, uint64_t seed, const int* row_live, int* out) {
    GUARD(((OpsHandle*)h)->begin().sample(*T(logits), temperature, streams, steps, seed, row_live, out))
}
FR_API int friday_ops_plan(void* h, int64_t rows, int64_t n, int64_t k, int* swapped, int* bn, int* splits) {
    GUARD({
        bool s = false;
        ((OpsHandle*)h)->ops->plan(rows, n, k, &s, bn, splits);
        *swapped = s ? 1 : 0;
    })
}
FR_API int friday_ops_decode_splits(void* h, int n_seqs, int nq, int nkv, int hd, int max_kv_len, int* splits) {
    GUARD(*splits = ((OpsHandle*)h)->ops->decode_splits(n_seqs, nq, nkv, hd, max_kv_len))
}
FR_API int friday_ops_attention_splits(void* h, int64_t rows, int nq, int max_kv_len, int* splits) {
    GUARD(*splits = ((OpsHandle*)h)->ops->attention_splits(rows, nq, max_kv_len))
}
FR_API int friday_ops_tensor_core_ok(void* h, const FridayTensor* x, const FridayTensor* w, const FridayTensor* out, int* ok) {
    GUARD(*ok = ((OpsHandle*)h)->ops->tensor_core_ok(*T(x), *T(w), *T(out), nullptr) ? 1 : 0)
}
FR_API int friday_ops_info(void* h, const char** json) {
    GUARD({
        Ops& ops = *((OpsHandle*)h)->ops;
        Json j = Json::object();
        j.set("sm_count", Json(ops.sm_count()));
        j.set("fusion", Json(ops.fusion_enabled()));
        j.set("launches", Json((int64_t)ops.launches()));
        j.set("status_word", Json((int64_t)(intptr_t)ops.status_word()));
        *json = hand_back(j.dump());
    })
}
FR_API int friday_ops_check_status(void* h) { GUARD(((OpsHandle*)h)->ops->check_status()) }
