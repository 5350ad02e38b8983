// A decoder put together from a ModelSpec: token table, blocks, final norm, head.
//
// It knows nothing of any architecture: the specification says which parts there are and
// in which order they run.  `run` takes the tokens of one pass as rows, sends them through
// the program, and returns the residual stream; `logits` applies the final norm and the
// head to chosen rows only (the reference does this for one row: transformer.cpp:1077-1113).
#pragma once
#include <map>
#include <memory>
#include <vector>

#include "friday/base.h"
#include "friday/ops.h"
#include "friday/parts.h"
#include "friday/weights.h"

namespace friday {

// The loader, for any tree of parts.  plan_storage compares the declared tensors with the source (one WeightsError
// for everything that does not fit) and decides in which dtype each is kept; load_params allocates device memory,
// stacks what the parts asked to have stacked, copies, and returns the bytes held.  Parts are finalized by the caller.
struct StoredParam { Part::Named param; DType dtype; };
std::vector<StoredParam> plan_storage(const std::vector<Part::Named>& declared, const WeightSource& source, DType compute,
                                      const std::vector<std::string>& ignorable);
size_t load_params(const std::vector<StoredParam>& plan, WeightSource& source, Ops& ops);

class DecoderModel {
public:
    // Builds the parts (host only: no device memory is touched until load()).
    DecoderModel(const ModelSpec& spec, DType dtype);

    ModelSpec spec;
    BuildEnv env;
    std::vector<std::unique_ptr<Block>> layers;
    std::unique_ptr<Norm> final_norm;
    std::map<int, int> owners;                     // cache entry -> program entry that writes it
    Tensor embedding, head, head_bias;

    // Every tensor the model needs, by full name (a layer that the run order names twice has its tensors once).
    std::vector<Part::Named> named_params();
    // Compares names and shapes with the source (one WeightsError for everything) and decides in which dtype every
    // tensor is kept (the storage rule of weights.h; members of a stacked tensor share its dtype).  Host only.
    std::vector<StoredParam> plan_storage(const WeightSource& source);
    // plan_storage, then allocates, copies and finalizes.
    void load(WeightSource& source, Ops& ops);
    std::map<int, CacheRequest> cache_requests() const;
    size_t parameter_bytes() const { return parameter_bytes_; }

    struct RunOut {
        Tensor x;
        bool has_normed = false;
        Rows normed;               // the final norm of every row, if asked for and produced on the way
    };
    // views: one cache view per program entry.  Results of a layer live in one of two arenas in turn, so a layer's
    // working memory is taken back when the layer after the next starts; what must outlive the pass comes from
    // the arena that is current when run() is called.
    RunOut run(Ops& ops, const StepContext& ctx, const std::vector<CacheView>& views, bool with_final_norm,
               Arena* layer_arenas[2]);
    // fp32 logits [n, vocab] of rows `rows` (device int32; null: all rows) of x.
    Tensor logits(Ops& ops, const Tensor& x, const int* rows, int64_t n_rows, const Rows* normed);

private:
    class Root;
    std::unique_ptr<Part> root_;                   // owns the token table, the head and its bias
    size_t parameter_bytes_ = 0;
};

}  // namespace friday
