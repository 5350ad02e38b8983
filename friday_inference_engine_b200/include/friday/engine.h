// friday::Engine: the public entry point, in the manner of the reference's friday::Engine
// (engine.h:19-72): options in, then step / prefill / generate; callers never handle
// device memory unless they ask for it.
//
// Where the reference has an option, its name and meaning are kept: `model_path`,
// `max_ctx` (tokens one sequence can hold, default 2048: engine.h:22).  Its options for
// CPU offload, a VRAM limit and quantized KV (`vram_gb`, `cpu_threads`, `backend`,
// `kv_cache`) have nothing to act on here and are not offered.  New ones: `dtype`,
// `max_batch` (sequences alive at once), `max_tokens` (cache capacity), and a
// random-weights mode from a configuration and a seed.
//
//     friday::EngineOptions opt;
//     opt.model_path = "/models/qwen2.5-7b";
//     friday::Engine engine(opt);
//     auto out = engine.generate({{1, 2, 3}, {4, 5}}, friday::GenerateOptions());
//
// One step function serves everything: a batch of sequences, each with its next tokens
// (whole prompts of unequal lengths, or one token each, or a mix), run as ONE batch from
// the cache, with logits for the places that were asked for.
#pragma once
#include <stdint.h>

#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "friday/base.h"
#include "friday/json.h"

namespace friday {

struct EngineOptions {
    std::string model_path;          // folder with config.json and model.safetensors (or an index and its shards)
    std::string config_json;         // instead of model_path: config.json's text, random weights
    uint64_t seed = 0;               // of the random weights
    std::string dtype = "bfloat16";  // "bfloat16": what serving uses; "float32": everything in true 32-bit
    int max_ctx = 2048;              // tokens one sequence can hold
    int max_batch = 8;               // sequences alive at once
    int64_t max_tokens = 0;          // cache capacity in tokens; 0: max_batch * max_ctx (in pages)
    int device = 0;
    int prefill_chunk = 2560;        // most tokens of one sequence per pass (ten 256-row tiles of a prompt's products)
    bool cuda_graphs = true;         // decode steps of generate() are captured once and replayed
    bool random_on_device = true;    // random weights are drawn on the device (fast); false: on the host
    bool profile = false;            // event-bracketed time per kind of kernel and host time per step (see profile())
};

struct Generation {
    std::vector<int> tokens;
    std::string finish_reason;       // "stop" | "length" | "context"
};

struct GenerateOptions {
    int max_new_tokens = 100;        // the reference's fixed budget (main.cpp:328)
    float temperature = 0.0f;        // 0: greedy, the first maximum wins (main.cpp:90-101)
    uint64_t seed = 0;               // of the sampler
    std::vector<int> stop_token_ids; // a sequence that draws one ends; the id is not kept (main.cpp:331-332)
    bool ignore_eos = false;
    // called after every step with the requests that took part and the ids they drew
    std::function<void(const std::vector<int>& requests, const std::vector<int>& tokens)> on_step;
};

struct StepBatch {
    std::vector<int> slots;                      // one per sequence (alloc_slot)
    std::vector<std::vector<int>> tokens;        // for each its next token ids
    std::vector<std::vector<int>> want;          // for each the places among these tokens whose logits are asked for
};

// Where the time of the steps since the last call went (options.profile).
struct Profile {
    long long steps = 0;
    double host_ms = 0;              // wall time inside step calls, launches and copies included
    double product_ms = 0, attention_ms = 0, other_ms = 0;      // device time between events around each kernel
    long long product_calls = 0, attention_calls = 0, other_calls = 0;
};

class Decoder;

class Engine {
public:
    explicit Engine(const EngineOptions& options);
    ~Engine();
    Engine(const Engine&) = delete;

    int vocabSize() const;
    int maxContext() const;
    int maxBatch() const;
    std::string summary() const;
    const Json& config() const;                  // the typed configuration
    std::string architecture() const;
    size_t parameterBytes() const;
    size_t cacheBytes() const;

    int allocSlot();
    void freeSlot(int slot);
    int slotLength(int slot) const;

    // Runs the batch and writes fp32 logits [sum of want sizes][vocab] to `logits`, in the order of the
    // sequences and, within one, of `want`.  logits_on_device: `logits` is device memory (else host).
    // Returns the number of rows written.
    size_t step(const StepBatch& batch, float* logits, bool logits_on_device = false);

    // Single-sequence conveniences with the reference's meaning (engine.h:44-54): one token at position `pos`, or
    // n tokens at pos .. pos+n-1 (logits of the last one).  Position 0 starts a new sequence.
    void step(int token, int pos, float* logits);
    void prefill(const int* tokens, int n, int pos, float* logits);

    std::vector<Generation> generate(const std::vector<std::vector<int>>& prompts, const GenerateOptions& options);

    // Decoding of the sequences in `slots`, one token each per step, from buffers that stay on the device.
    std::unique_ptr<Decoder> decoder(const std::vector<int>& slots, const std::vector<int>& first_tokens,
                                     float temperature = 0.0f, uint64_t seed = 0, const std::vector<int>& streams = {},
                                     const std::vector<int>& steps_done = {});
    void keepDecoder(std::unique_ptr<Decoder> d);      // its buffers and captured steps serve the next batch of its size

    void check();                                // raises KernelError if a kernel gave up on one of its bounded waits
    Profile profile();                           // and clears the counters
    void* stream() const;                        // the cudaStream_t everything runs on
    long long launches() const;                  // kernel launches so far (graph replays count what they hold)
    int* statusWord() const;                     // device address of the word that check() reads
    int64_t cacheHeldTokens() const;
    int cacheHeldSlots() const;
    int cacheHeldPages(int group) const;
    int cacheGroups() const;
    std::string cacheLayout() const;             // JSON: groups (entries, window, pages) and states

    struct Impl;
    Impl* impl() { return impl_.get(); }

private:
    std::unique_ptr<Impl> impl_;
};

// Decoding one token per sequence, step after step, with everything the kernels read in buffers that keep their
// addresses, so that the step can be captured once in a CUDA graph and replayed (the reference captures its layer
// stack the same way and lets kernels read the position from device memory: transformer.cpp:1465-1483,
// attention_kernels.cu:33).  A step is: embedding of each row's token, the model's program over the cache, final
// norm and head for every row, the sampler, and `advance` (the chosen token becomes the row's next input; position
// and length grow by one).  A row whose sequence has ended is marked dead: kernels skip it.
class Decoder {
public:
    virtual ~Decoder() {}
    virtual int rows() const = 0;
    // One step.  tokens: each row's input token (dead rows: anything), or null to go on with the tokens that the
    // previous step chose.
    virtual void step(const int* tokens) = 0;
    virtual std::vector<int> sampled() = 0;                      // waits for the step
    virtual void logits(float* out, bool on_device) = 0;         // the last step's logits [rows, vocab]
    virtual void retire(int row) = 0;                            // the caller frees its slot
    virtual long long launchesPerStep() const = 0;
    virtual int graphsCaptured() const = 0;
    virtual int bound() const = 0;                               // the length bound of the step in use
};

// The generation loop alone, with the step function, the sampler and the slot book-keeping handed in, so that its
// decisions can be tested without a model (generate.cpp).
struct LoopHooks {
    std::function<void(const std::vector<int>& slots, const std::vector<std::vector<int>>& tokens,
                       const std::vector<std::vector<int>>& want)> step;
    // ids for the rows of the last step's logits; streams: request numbers; steps: tokens drawn so far
    std::function<std::vector<int>(const std::vector<int>& streams, const std::vector<int>& steps)> sample;
    std::function<int()> alloc_slot;
    std::function<void(int)> free_slot;
    // optional: a decoder for the one-token steps
    struct Rows {
        std::function<std::vector<int>(const std::vector<int>& tokens)> step;
        std::function<void(int)> retire;
        std::function<void()> close;
    };
    std::function<Rows(const std::vector<int>& slots, const std::vector<int>& first_tokens,
                       const std::vector<int>& streams, const std::vector<int>& steps_done)> decoder;
};
std::vector<Generation> generate_loop(const std::vector<std::vector<int>>& prompts, const LoopHooks& hooks, int max_batch,
                                      int max_context, int vocab_size, const GenerateOptions& options);

// A model folder from a configuration and a seed (weights.h); here so that users of the engine header find it.
void write_random_model(const std::string& dir, const Json& config_json, uint64_t seed, const std::string& dtype,
                        int shards);

}  // namespace friday
