// What an Engine holds (internal): device, stream, operations, model, cache, the step function and the decoders.
#pragma once
#include <chrono>
#include <map>
#include <memory>
#include <vector>

#include "friday/cache.h"
#include "friday/config.h"
#include "friday/engine.h"
#include "friday/model.h"
#include "friday/ops.h"

namespace friday {

// Pinned host memory for the small arrays that a pass sends to the device in one copy.
class PinnedRing {
public:
    ~PinnedRing();
    // A buffer of at least `bytes`, free to be overwritten (the copy that last used it has finished).
    void* next(size_t bytes);
    void sent(cudaStream_t stream);          // marks the buffer handed out last as in flight on `stream`

private:
    struct Slot { void* p = nullptr; size_t cap = 0; cudaEvent_t ev = nullptr; bool busy = false; };
    Slot slots_[4];
    int next_ = 0, last_ = 0;
};

// The step function: a batch of sequences, each with its next tokens, run as ONE batch from the cache; logits
// come back for the places that were asked for.
//
// A step is either the start of sequences (whole prompts of unequal lengths, or any number of further tokens for
// sequences that already hold some) or one token for each, or a mix: the same code runs them all, because every
// row of the batch carries its own sequence and position and the kernels read only that.  Rows are the tokens of
// all sequences laid end to end, as the reference lays a prompt's tokens out as [T][.] rows
// (transformer.cpp:1129-1149); there are no padding rows in a pass, so padding cannot change a result.
//
// Long inputs are cut into passes of at most `chunk` tokens per sequence (the reference cuts prompts at 512:
// transformer.cpp:1369).  A pass runs all layers; the next pass finds the earlier tokens in the cache.  The cut
// changes no result beyond rounding.
//
// Host-side layout of a pass (int32, sent to the device in one copy):
//     tokens[rows] | row_seq[rows] | row_pos[rows] | want_rows[n] | seq_start[n_seqs] | seq_qlen[n_seqs] |
//     seq_pos0[n_seqs] | seq_slots[n_seqs] | per group: table[n_seqs][width]
class Stepper {
public:
    Stepper(DecoderModel& model, Cache& cache, Ops& ops, int chunk);
    void check(const StepBatch& b) const;
    // Returns the rows written to `out` ([rows][vocab] fp32; device or host memory).
    size_t step(const StepBatch& b, float* out, bool out_on_device);
    // The logits of the last step stay on the device until the next one: [rows, vocab], in the order of the result.
    Tensor last_logits;
    size_t last_upload_bytes = 0;
    double last_queue_ms = 0;      // host time of the last step until all its launches were queued

private:
    DecoderModel& model_;
    Cache& cache_;
    Ops& ops_;
    int chunk_;
    Arena pass_, layer_a_, layer_b_, keep_;
    PinnedRing ring_;
};

struct Engine::Impl {
    EngineOptions options;
    DType dtype;
    int device = 0;
    cudaStream_t stream = nullptr;
    Json typed_config;
    std::string arch_name;
    std::unique_ptr<Ops> ops;
    std::unique_ptr<DecoderModel> model;
    std::unique_ptr<Cache> cache;
    std::unique_ptr<Stepper> stepper;
    int max_ctx = 0, max_batch = 0;
    int single = -1;                                     // slot of the single-sequence conveniences
    std::map<int, std::unique_ptr<Decoder>> kept;        // batch size -> a decoder that is not in use
    std::vector<float> host_logits;                      // for generate(): rows are sampled on the device
    Profile prof;
    ~Impl();
};

std::unique_ptr<Decoder> make_device_decoder(Engine::Impl& e, const std::vector<int>& slots,
                                             const std::vector<int>& first_tokens, float temperature, uint64_t seed,
                                             const std::vector<int>& streams, const std::vector<int>& steps_done);
// Re-arms a kept decoder for another batch of its size; false if it cannot serve it.
bool reset_device_decoder(Decoder& d, const std::vector<int>& slots, const std::vector<int>& first_tokens,
                          float temperature, uint64_t seed, const std::vector<int>& streams,
                          const std::vector<int>& steps_done);

}  // namespace friday
