// What a model is made of, and how a new kind of part or a new architecture is added.
//
// A model is described as data (ModelSpec): a token table, a list of layers (each a
// PartSpec naming a registered block with its constants and sub-parts), the order in
// which layers run (`program`, which may name a layer twice or let a call read the cache
// entry another call wrote), a final norm and a head.  Everything below the architecture
// (loader, cache, step function) works from the ModelSpec and never asks which model it
// is in; no part refers to a model.
//
// Categories of parts and what each must offer:
//
//   Norm         forward(ops, x[rows, width]) -> tensor of the same shape.  A plain RMSNorm
//                also answers as_rmsnorm(), so that the product before it can begin it.
//   Position     a rotary part answers rotary() with its table of denominators; the mixer
//                hands that to the kernel that rotates q and k.  Any other encoding answers
//                false and changes q and k itself in apply().
//   Mixer        cache_request(): keys and values per position, a fixed-size state per
//                sequence, or nothing;  forward(ops, h, residual, ctx, view, then) ->
//                residual + mix(h).
//   FeedForward  forward(ops, h, residual, ctx, then) -> residual + f(h).
//   Block        cache_request() (its mixer's); forward(ops, x, normed, ctx, view, then).
//
// `h` is a Rows: either a tensor or rows whose RMSNorm a product has begun and the next
// product finishes (ops.h); a part that cannot take the latter calls ops.materialize(h).
// `then` names the norm that will be applied to the part's result (or null).  A part may
// ignore it and return `PartOut{x}`; a part that ends in a product passes it to
// ops.linear_norm and returns the normed rows too, which saves a kernel per layer.
//
// A part owns its parameters: it declares them by local tensor name (declare) and adopts
// its sub-parts under a prefix; the loader walks that tree, so a part never sees a file.
// finalize() runs once when every parameter is set (to stack matrices, build tables).
//
// Adding a part: derive from the category's class, then
//     static friday::PartRegistrar reg("mixer", "my_mixer", [](const PartSpec& s, const BuildEnv& e) { return new MyMixer(s, e); });
// in a library that the process loads (load_plugin, or linked in).  Adding an
// architecture: register_architecture({name, read_config, build_spec}) (config.h).
#pragma once
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "friday/base.h"
#include "friday/json.h"

namespace friday {

class Ops;
struct Rows;
struct StepContext;

struct PartSpec {
    std::string kind;                           // a registered name of the part's category
    Json params = Json::object();               // sizes and constants
    std::string prefix;                         // what its tensor names start with inside its parent
    std::map<std::string, PartSpec> parts;      // sub-parts by role ("position", "mixer", ...)

    PartSpec() {}
    PartSpec(const std::string& k, const Json& p = Json::object(), const std::string& pre = "")
        : kind(k), params(p), prefix(pre) {}
    const PartSpec& part(const std::string& role) const;            // ConfigError if absent
};

struct LayerCall {
    int layer = 0;          // index into ModelSpec::layers; a layer may be named by several entries
    int cache = -1;         // cache entry that the layer's mixer uses in this call; -1: none
    bool write = true;      // false: read an entry that an earlier call filled
};

struct ModelSpec {
    std::string architecture;
    int64_t vocab_size = 0, width = 0, max_positions = 0;
    std::string embedding;                      // tensor name of the token table [vocab, width]
    std::vector<PartSpec> layers;               // category "block"
    std::vector<LayerCall> program;
    PartSpec final_norm;
    std::string head;                           // tensor name of the head [vocab, width]; empty: the token table
    std::string head_bias;                      // tensor name of a bias [vocab] added to the logits; empty: none
    std::vector<std::string> ignorable;         // tensors a checkpoint may carry that the model does not use
    double embed_scale = 1.0;                   // token rows are multiplied by this
    double logit_scale = 1.0;                   // logits are multiplied by this
    double logit_softcap = 0.0;                 // > 0: logits = cap * tanh(logits / cap)

    // cache entry -> index of the program entry that writes it; checks the program.
    std::map<int, int> cache_entries() const;
};

// ---- what a mixer may ask of the cache
struct CacheRequest {
    enum Kind { None, KV, State } kind = None;
    int n_kv_heads = 0, head_dim = 0, window = 0;    // KV: keys and values for every position, or the last `window`
    std::vector<int64_t> state_shape;                // State: a tensor of this shape per sequence, zero at its start
    DType state_dtype = DType::F32;
    static CacheRequest kv(int n_kv_heads, int head_dim, int window = 0);
    static CacheRequest state(const std::vector<int64_t>& shape, DType dtype = DType::F32);
};

// ---- what the cache hands a mixer for one layer call
struct CacheView {
    CacheRequest::Kind kind = CacheRequest::None;
    bool write = true;
    // KV: pools [pages][page_size][kv heads][head_dim] of this entry and this step's block table on the device
    void* k_pool = nullptr;
    void* v_pool = nullptr;
    int pool_pages = 0;
    const int* block_table = nullptr;      // [n_seqs][table_width], -1 where the sequence holds no page
    int table_width = 0, page_size = 0, window = 0, n_kv_heads = 0, head_dim = 0;
    DType dtype = DType::F32;
    // State: state[slot] is the sequence's own tensor
    Tensor state;                          // [slots, ...]
    const int* seq_slots = nullptr;        // device: slot of every sequence of the step
};

// ---- the geometry of one pass of the step function; parts read it, nothing writes it once it is built
struct StepContext {
    int rows = 0, n_seqs = 0, max_q_len = 0, max_kv_len = 0;
    bool decode = false;                   // every sequence brings exactly one token
    std::vector<int> slots, q_lens, kv_lens;                 // host: per sequence
    // device, int32: per row, then per sequence
    const int* tokens = nullptr;
    const int* row_seq = nullptr;          // sequence of the step that a row belongs to (negative: a dead row)
    const int* row_pos = nullptr;          // position of the row's token in its sequence
    const int* seq_start = nullptr;        // first row of each sequence
    const int* seq_qlen = nullptr;
    const int* seq_pos0 = nullptr;         // position of each sequence's first row
};

struct BuildEnv {
    int64_t width = 0;       // of the residual stream
    DType dtype = DType::F32;
};

struct ParamDecl {
    std::vector<int64_t> shape;
    bool integer = false;    // kept as int32; otherwise in the activation dtype unless stored in 32-bit
    bool one = false;        // random-weights mode: 1 + N(0, 0.02) (norm weights) instead of N(0, 0.02)
    // A parameter may be loaded straight into rows of a larger tensor that the part declared with
    // declare_stacked (q, k and v under one another; gate and up row by row in turn): row r of the parameter
    // becomes row row0 + r * row_step of `into`.  The stacked tensor is 32-bit if any of its members is stored so.
    std::string into;
    int64_t row0 = 0, row_step = 1;
    ParamDecl& stack(const std::string& name, int64_t first_row, int64_t step = 1) {
        into = name;
        row0 = first_row;
        row_step = step;
        return *this;
    }
};

class Part {
public:
    virtual ~Part() {}
    std::string prefix;
    BuildEnv env;

    ParamDecl& declare(const std::string& name, const std::vector<int64_t>& shape, bool integer = false, bool one = false);
    void declare_stacked(const std::string& name, int64_t rows, int64_t cols) { stacked.emplace_back(name, std::vector<int64_t>{rows, cols}); }
    void hold(std::shared_ptr<void> memory) { memory_.push_back(std::move(memory)); }      // keeps device memory alive
    template <class P> P* adopt(const std::string& prefix, P* child) {
        children_.emplace_back(prefix, std::unique_ptr<Part>(child));
        return child;
    }
    void set_tensor(const std::string& name, const Tensor& t) { tensors[name] = t; }
    const Tensor& tensor(const std::string& name) const;                 // KernelError if unset
    virtual void finalize(Ops& ops);                                       // default: the children's

    struct Named { std::string name; Part* owner; std::string local; ParamDecl decl; };
    void named_params(const std::string& prefix, std::vector<Named>& out);
    const std::vector<std::pair<std::string, std::unique_ptr<Part>>>& children() const { return children_; }

    std::map<std::string, Tensor> tensors;         // set by the loader
    std::vector<std::pair<std::string, ParamDecl>> params;
    std::vector<std::pair<std::string, std::vector<int64_t>>> stacked;

protected:
    explicit Part(const BuildEnv& e) : env(e) {}

private:
    std::vector<std::pair<std::string, std::unique_ptr<Part>>> children_;
    std::vector<std::shared_ptr<void>> memory_;
};

class Norm : public Part {
public:
    using Part::Part;
    virtual Tensor forward(Ops& ops, const Tensor& x) = 0;
    virtual bool as_rmsnorm(Tensor* weight, float* eps) const { return false; }
};

class Position : public Part {
public:
    using Part::Part;
    // A rotary encoding: pairs (i, i + rotary_dim/2) of every q and k head turn by pos / denominators[i].
    virtual bool rotary(const float** denominators, int* rotary_dim) const { return false; }
    // Any other encoding changes q and k inside qkv [rows, (n_heads + 2 n_kv_heads) * head_dim] itself.
    virtual void apply(Ops& ops, Tensor& qkv, const StepContext& ctx, int n_heads, int n_kv_heads, int head_dim) {}
};

struct PartOut;

class Mixer : public Part {
public:
    using Part::Part;
    virtual CacheRequest cache_request() const { return CacheRequest(); }
    virtual PartOut forward(Ops& ops, const Rows& h, const Tensor& residual, const StepContext& ctx,
                            const CacheView& view, Norm* then) = 0;
};

class FeedForward : public Part {
public:
    using Part::Part;
    virtual PartOut forward(Ops& ops, const Rows& h, const Tensor& residual, const StepContext& ctx, Norm* then) = 0;
};

class Block : public Part {
public:
    using Part::Part;
    virtual CacheRequest cache_request() const { return CacheRequest(); }
    virtual Norm* first_norm() { return nullptr; }       // the norm the block begins with, if the block before may apply it
    // normed: first_norm of x if the caller has it already (else null); then: the norm that follows this block.
    virtual PartOut forward(Ops& ops, const Tensor& x, const Rows* normed, const StepContext& ctx,
                            const CacheView& view, Norm* then) = 0;
};

// ---- the registry of parts
typedef std::function<Part*(const PartSpec&, const BuildEnv&)> PartFactory;
void register_part(const std::string& category, const std::string& kind, PartFactory factory);
Part* build_part(const std::string& category, const PartSpec& spec, const BuildEnv& env);     // ConfigError if unknown
std::vector<std::string> registered_parts(const std::string& category);
template <class P> P* build(const std::string& category, const PartSpec& spec, const BuildEnv& env) {
    Part* p = build_part(category, spec, env);
    P* typed = dynamic_cast<P*>(p);
    if (!typed) {
        delete p;
        throw ConfigError("part '" + spec.kind + "' is not a " + category);
    }
    return typed;
}
struct PartRegistrar {
    PartRegistrar(const char* category, const char* kind, PartFactory f) { register_part(category, kind, std::move(f)); }
};

// Loads a shared library whose static registrars add parts or architectures.
void load_plugin(const std::string& path);

}  // namespace friday
