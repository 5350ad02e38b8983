// The device decoder (engine.h, class Decoder): one-token steps from long-lived buffers, captured in CUDA graphs.
//
// Between steps the host only reserves cache pages (a table row changes every 64 tokens) and, if the caller drives
// the tokens itself (generation with stop tokens, replayed traces), writes the step's tokens.  It uses the same
// model, cache, kernels and page tables as the step function; only the buffers are long-lived.
//
// Launch shapes depend on how long the longest sequence may be (how many ways its keys are split), so a captured
// step serves lengths up to a bound; when a sequence outgrows it, the next bound's step is used.  Bounds double
// from 1,024 tokens.  The first step at a bound runs eagerly: it loads what it needs and sizes the working memory,
// so that the capture that follows allocates nothing.  Working memory is handed out in the same order every step,
// so addresses repeat; should an arena have had to grow, every captured step is dropped and captured again.
#include <string.h>

#include <algorithm>

#include "engine/engine_impl.h"

namespace friday {

namespace {

class DeviceDecoder : public Decoder {
public:
    DeviceDecoder(Engine::Impl& e, const std::vector<int>& slots, const std::vector<int>& first_tokens, float temperature,
                  uint64_t seed, const std::vector<int>& streams, const std::vector<int>& steps_done)
        : e_(e), cache_(*e.cache), model_(*e.model), ops_(*e.ops), n_((int)slots.size()), pass_(e.stream, 1 << 20),
          layer_a_(e.stream, 1 << 20), layer_b_(e.stream, 1 << 20) {
        if (n_ <= 0) throw StepError("a decoder needs at least one sequence");
        use_graph_ = e.options.cuda_graphs && !e.options.profile;
        size_t ints = (size_t)10 * n_;
        for (const auto& g : cache_.groups) {
            table_off_.push_back(ints);
            ints += (size_t)n_ * g->width;
        }
        buf_ = DeviceBuffer(ints * sizeof(int), true);
        int* b = buf_.as<int>();
        tokens_ = b;
        row_seq_ = b + n_;
        row_pos_ = b + 2 * n_;
        kv_len_ = b + 3 * n_;
        sampled_ = b + 4 * n_;
        streams_ = b + 5 * n_;
        draws_ = b + 6 * n_;
        seq_start_ = b + 7 * n_;
        seq_qlen_ = b + 8 * n_;
        seq_slots_ = b + 9 * n_;
        temperature_ = DeviceBuffer(n_ * sizeof(float));
        cuda_check(cudaMallocHost(&pin_in_, n_ * sizeof(int)), "cudaMallocHost");
        cuda_check(cudaMallocHost(&pin_out_, n_ * sizeof(int)), "cudaMallocHost");
        cuda_check(cudaEventCreateWithFlags(&copied_, cudaEventDisableTiming), "cudaEventCreate");
        tables_host_.resize(cache_.groups.size());
        arm(slots, first_tokens, temperature, seed, streams, steps_done);
    }

    ~DeviceDecoder() override {
        drop_graphs();
        if (copied_) cudaEventDestroy(copied_);
        if (pin_in_) cudaFreeHost(pin_in_);
        if (pin_out_) cudaFreeHost(pin_out_);
    }

    // (Re)starts the decoder on a batch of its size.  The buffers keep their addresses, so captured steps stay valid;
    // they are captured again only if the sampler's seed changes (a kernel argument).
    void arm(const std::vector<int>& slots, const std::vector<int>& first_tokens, float temperature, uint64_t seed,
             const std::vector<int>& streams, const std::vector<int>& steps_done) {
        if ((int)slots.size() != n_ || (int)first_tokens.size() != n_) throw StepError("decoder: one first token per slot");
        for (int s : slots)
            if (!cache_.slots.holds(s)) throw StepError(format("decoder: slot %d is not held", s));
        slots_ = slots;
        live_.assign((size_t)n_, 1);
        std::vector<int> host((size_t)10 * n_);
        for (int i = 0; i < n_; ++i) {
            host[i] = first_tokens[i];
            host[n_ + i] = i;
            host[2 * n_ + i] = cache_.lens[slots[i]];
            host[3 * n_ + i] = cache_.lens[slots[i]] + 1;
            host[4 * n_ + i] = 0;
            host[5 * n_ + i] = streams.empty() ? i : streams[i];
            host[6 * n_ + i] = steps_done.empty() ? 0 : steps_done[i];
            host[7 * n_ + i] = i;
            host[8 * n_ + i] = 1;
            host[9 * n_ + i] = slots[i];
        }
        // Copies go through the engine's stream: a plain cudaMemcpy from pageable memory may return before the data has
        // reached the device, and nothing would order the stream's kernels behind it.
        cuda_check(cudaMemcpyAsync(buf_.get(), host.data(), host.size() * sizeof(int), cudaMemcpyHostToDevice, e_.stream),
                   "cudaMemcpyAsync");
        std::vector<float> temp((size_t)n_, temperature);
        cuda_check(cudaMemcpyAsync(temperature_.get(), temp.data(), temp.size() * sizeof(float), cudaMemcpyHostToDevice,
                                   e_.stream), "cudaMemcpyAsync");
        // the seed is a kernel argument, and a mixer with state of its own may address it from the host
        if (seed != seed_ || !armed_ || !cache_.states.empty()) {
            seed_ = seed;
            drop_graphs();
        }
        armed_ = true;
        for (size_t g = 0; g < cache_.groups.size(); ++g) {
            tables_host_[g].clear();
            cache_.table_rows((int)g, slots_, tables_host_[g]);
            cuda_check(cudaMemcpyAsync(buf_.as<int>() + table_off_[g], tables_host_[g].data(),
                                       tables_host_[g].size() * sizeof(int), cudaMemcpyHostToDevice, e_.stream), "cudaMemcpyAsync");
        }
        cuda_check(cudaStreamSynchronize(e_.stream), "cudaStreamSynchronize");      // the host vectors above may go now
        int longest = 0;
        for (int s : slots_) longest = std::max(longest, cache_.lens[s]);
        set_bound(bound_for(longest + 1));
        std::vector<const int*> tables;
        for (size_t g = 0; g < cache_.groups.size(); ++g) tables.push_back(buf_.as<int>() + table_off_[g]);
        views_.clear();
        for (const auto& call : model_.spec.program)
            views_.push_back(call.cache < 0 ? CacheView() : cache_.view(call.cache, call.write, tables, seq_slots_));
        ctx_ = StepContext();
        ctx_.rows = n_;
        ctx_.n_seqs = n_;
        ctx_.max_q_len = 1;
        ctx_.decode = true;
        ctx_.slots = slots_;
        ctx_.q_lens.assign((size_t)n_, 1);
        ctx_.tokens = tokens_;
        ctx_.row_seq = row_seq_;
        ctx_.row_pos = row_pos_;
        ctx_.seq_start = seq_start_;
        ctx_.seq_qlen = seq_qlen_;
        ctx_.seq_pos0 = row_pos_;                 // one row per sequence: the row's position is the sequence's
        set_bound(bound_);
        pending_copy_ = false;
    }

    int rows() const override { return n_; }
    long long launchesPerStep() const override { return launches_per_step_; }
    int graphsCaptured() const override { return (int)graphs_.size(); }
    int bound() const override { return bound_; }

    void step(const int* tokens) override {
        if (!e_.options.profile) return step_now(tokens);
        const auto t0 = std::chrono::steady_clock::now();       // profile: a decode step counts like a call of the step function
        step_now(tokens);
        e_.prof.host_ms += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        e_.prof.steps += 1;
    }

    void step_now(const int* tokens) {
        cuda_check(cudaSetDevice(e_.device), "cudaSetDevice");
        sync_tables();
        int longest = 0;
        for (int i = 0; i < n_; ++i)
            if (live_[i]) longest = std::max(longest, cache_.lens[slots_[i]]);
        const int need = bound_for(longest + 1);
        if (need != bound_) set_bound(need);
        if (tokens) {
            if (pending_copy_) cuda_check(cudaEventSynchronize(copied_), "cudaEventSynchronize");   // the copy before has read the buffer
            memcpy(pin_in_, tokens, n_ * sizeof(int));
            cuda_check(cudaMemcpyAsync(tokens_, pin_in_, n_ * sizeof(int), cudaMemcpyHostToDevice, e_.stream), "cudaMemcpyAsync");
            cuda_check(cudaEventRecord(copied_, e_.stream), "cudaEventRecord");
            pending_copy_ = true;
        }
        if (!graphs_.empty() && generation() != graph_generation_) drop_graphs();      // working memory has moved or will
        auto it = graphs_.find(bound_);
        if (!use_graph_) {
            body();
        } else if (it != graphs_.end()) {
            cuda_check(cudaGraphLaunch(it->second, e_.stream), "cudaGraphLaunch");
            ops_.add_launches(launches_per_step_);
            logits_ = graph_logits_.at(bound_);        // where this bound's captured step leaves them
        } else if (!eager_done_.count(bound_)) {
            const long long before = ops_.launches();
            body();                                   // loads libraries, sizes the working memory
            launches_per_step_ = ops_.launches() - before;
            eager_done_.insert(bound_);
        } else {
            capture();
            cuda_check(cudaGraphLaunch(graphs_.at(bound_), e_.stream), "cudaGraphLaunch");
            ops_.add_launches(launches_per_step_);
        }
        std::vector<int> live_slots, ones;
        for (int i = 0; i < n_; ++i)
            if (live_[i]) {
                live_slots.push_back(slots_[i]);
                ones.push_back(1);
            }
        cache_.commit(live_slots, ones);
    }

    std::vector<int> sampled() override {
        cuda_check(cudaMemcpyAsync(pin_out_, sampled_, n_ * sizeof(int), cudaMemcpyDeviceToHost, e_.stream), "cudaMemcpyAsync");
        cuda_check(cudaStreamSynchronize(e_.stream), "cudaStreamSynchronize");
        return std::vector<int>(pin_out_, pin_out_ + n_);
    }

    void logits(float* out, bool on_device) override {
        if (!logits_.defined()) throw StepError("the decoder has not run a step yet");
        cuda_check(cudaMemcpyAsync(out, logits_.data, logits_.bytes(), on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost,
                                   e_.stream), "cudaMemcpyAsync");
        cuda_check(cudaStreamSynchronize(e_.stream), "cudaStreamSynchronize");
    }

    void retire(int row) override {
        if (row < 0 || row >= n_) throw StepError(format("decoder: no row %d", row));
        live_[row] = 0;
        cuda_check(cudaMemsetAsync(row_seq_ + row, 0xFF, sizeof(int), e_.stream), "cudaMemsetAsync");     // -1: kernels skip the row
    }

private:
    int bound_for(int length) const {
        int b = 1024;
        while (b < length) b *= 2;
        return std::min(b, std::max(cache_.max_seq_tokens, 1));
    }
    uint64_t generation() const { return pass_.generation() + layer_a_.generation() + layer_b_.generation(); }
    void set_bound(int b) {
        bound_ = b;
        ctx_.max_kv_len = b;
        ctx_.kv_lens.assign((size_t)n_, b);
    }
    void drop_graphs() {
        for (auto& kv : graphs_) cudaGraphExecDestroy(kv.second);
        graphs_.clear();
        graph_logits_.clear();
    }

    void body() {
        pass_.reset();
        ops_.arena = &pass_;
        Arena* layers[2] = {&layer_a_, &layer_b_};
        DecoderModel::RunOut r = model_.run(ops_, ctx_, views_, true, layers);
        logits_ = model_.logits(ops_, r.x, nullptr, 0, r.has_normed ? &r.normed : nullptr);
        ops_.sample(logits_, temperature_.as<float>(), streams_, draws_, seed_, row_seq_, sampled_);
        ops_.advance(tokens_, sampled_, row_pos_, kv_len_, row_seq_, draws_, n_);
        ops_.arena = nullptr;
    }

    void capture() {
        pass_.reset();
        layer_a_.reset();
        layer_b_.reset();                                  // blocks are joined now, not inside the capture
        if (generation() != graph_generation_) {           // steps captured before the memory moved are stale
            drop_graphs();
            graph_generation_ = generation();
        }
        cuda_check(cudaStreamSynchronize(e_.stream), "cudaStreamSynchronize");
        pass_.frozen = layer_a_.frozen = layer_b_.frozen = true;
        const long long before = ops_.launches();
        cudaGraph_t graph = nullptr;
        cuda_check(cudaStreamBeginCapture(e_.stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
        try {
            body();
        } catch (...) {
            cudaStreamEndCapture(e_.stream, &graph);
            if (graph) cudaGraphDestroy(graph);
            pass_.frozen = layer_a_.frozen = layer_b_.frozen = false;
            ops_.arena = nullptr;
            throw;
        }
        pass_.frozen = layer_a_.frozen = layer_b_.frozen = false;
        cuda_check(cudaStreamEndCapture(e_.stream, &graph), "cudaStreamEndCapture");
        ops_.add_launches(before - ops_.launches());       // capturing launched nothing
        cudaGraphExec_t exec = nullptr;
        cudaError_t err = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        cuda_check(err, "cudaGraphInstantiate");
        graphs_[bound_] = exec;
        graph_logits_[bound_] = logits_;
    }

    void sync_tables() {
        std::vector<int> live_slots, ones;
        bool crossing = false;
        for (int i = 0; i < n_; ++i)
            if (live_[i]) {
                live_slots.push_back(slots_[i]);
                ones.push_back(1);
                if (cache_.lens[slots_[i]] % PAGE == 0) crossing = true;
            }
        if (!crossing) return;                       // nobody crosses into a new page: tables stand
        cache_.reserve(live_slots, ones);
        for (size_t g = 0; g < cache_.groups.size(); ++g) {
            const int width = cache_.groups[g]->width;
            std::vector<int> fresh;
            cache_.table_rows((int)g, slots_, fresh);
            for (int i = 0; i < n_; ++i)
                if (!live_[i])                       // a dead row keeps its stale table; nothing reads it
                    memcpy(&fresh[(size_t)i * width], &tables_host_[g][(size_t)i * width], width * sizeof(int));
            if (fresh != tables_host_[g]) {
                tables_host_[g] = fresh;
                int* staged = (int*)ring_.next(fresh.size() * sizeof(int));
                memcpy(staged, fresh.data(), fresh.size() * sizeof(int));
                cuda_check(cudaMemcpyAsync(buf_.as<int>() + table_off_[g], staged, fresh.size() * sizeof(int),
                                           cudaMemcpyHostToDevice, e_.stream), "cudaMemcpyAsync");
                ring_.sent(e_.stream);
            }
        }
    }

    Engine::Impl& e_;
    Cache& cache_;
    DecoderModel& model_;
    Ops& ops_;
    int n_;
    Arena pass_, layer_a_, layer_b_;
    PinnedRing ring_;
    DeviceBuffer buf_, temperature_;
    int *tokens_, *row_seq_, *row_pos_, *kv_len_, *sampled_, *streams_, *draws_, *seq_start_, *seq_qlen_, *seq_slots_;
    std::vector<size_t> table_off_;
    std::vector<std::vector<int>> tables_host_;
    std::vector<int> slots_;
    std::vector<char> live_;
    std::vector<CacheView> views_;
    StepContext ctx_;
    Tensor logits_;
    uint64_t seed_ = 0;
    bool armed_ = false, use_graph_ = true, pending_copy_ = false;
    int bound_ = 1024;
    std::map<int, cudaGraphExec_t> graphs_;
    std::map<int, Tensor> graph_logits_;
    std::set<int> eager_done_;
    uint64_t graph_generation_ = 0;
    long long launches_per_step_ = 0;
    int* pin_in_ = nullptr;
    int* pin_out_ = nullptr;
    cudaEvent_t copied_ = nullptr;
};

}  // namespace

std::unique_ptr<Decoder> make_device_decoder(Engine::Impl& e, const std::vector<int>& slots,
                                             const std::vector<int>& first_tokens, float temperature, uint64_t seed,
                                             const std::vector<int>& streams, const std::vector<int>& steps_done) {
    return std::unique_ptr<Decoder>(new DeviceDecoder(e, slots, first_tokens, temperature, seed, streams, steps_done));
}

bool reset_device_decoder(Decoder& d, const std::vector<int>& slots, const std::vector<int>& first_tokens,
                          float temperature, uint64_t seed, const std::vector<int>& streams,
                          const std::vector<int>& steps_done) {
    DeviceDecoder* dd = dynamic_cast<DeviceDecoder*>(&d);
    if (!dd || dd->rows() != (int)slots.size()) return false;
    dd->arm(slots, first_tokens, temperature, seed, streams, steps_done);
    return true;
}

}  // namespace friday
