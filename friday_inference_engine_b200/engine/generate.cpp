// The generation loop: prompts in, tokens out, for as many requests as there are.
//
// Requests are run in batches of at most `max_batch`, one batch after another.  A batch
// starts with all its prompts in one step; then every live sequence takes one token per
// step.  A sequence ends when it draws a stop token (which is not kept, as the reference
// prints nothing for it: main.cpp:331-332), when it has `max_new_tokens`, or when its
// context is full (main.cpp:335); it then leaves the batch, its slot goes back at once,
// and the others go on.  A prompt that would fill the context is refused before anything
// runs (main.cpp:319-322).
//
// The loop knows no kernels: it is given a step function, a sampler and the slot
// book-keeping (LoopHooks), so its decisions can be tested alone.  Stream numbers are the
// positions of the requests in `prompts`, so a request draws the same tokens whichever
// batch it lands in.
#include <algorithm>
#include <map>
#include <set>

#include "friday/engine.h"

namespace friday {

std::vector<Generation> generate_loop(const std::vector<std::vector<int>>& prompts, const LoopHooks& hooks, int max_batch,
                                      int max_context, int vocab_size, const GenerateOptions& opt) {
    std::set<int> stop;
    if (!opt.ignore_eos) stop.insert(opt.stop_token_ids.begin(), opt.stop_token_ids.end());
    for (size_t r = 0; r < prompts.size(); ++r) {
        const auto& p = prompts[r];
        if (p.empty()) throw GenerationError(format("request %zu has an empty prompt", r));
        if ((int)p.size() >= max_context)
            throw GenerationError(format("request %zu: the prompt (%zu tokens) is longer than the context (%d); use --ctx",
                                         r, p.size(), max_context));
        for (int t : p)
            if (t < 0 || t >= vocab_size)
                throw GenerationError(format("request %zu: token id %d is outside the vocabulary [0, %d)", r, t, vocab_size));
    }
    std::vector<Generation> results(prompts.size());
    if (opt.max_new_tokens <= 0) {
        for (auto& g : results) g.finish_reason = "length";
        return results;
    }
    if (max_batch <= 0) throw GenerationError("max_batch must be positive");

    // Books token `tok` for request r; true if the request goes on.
    auto settle = [&](int r, int tok) {
        Generation& g = results[r];
        if (tok < 0 || tok >= vocab_size)
            throw GenerationError(format("request %d: the sampler returned id %d, outside the vocabulary [0, %d) (a row of "
                                         "logits without a finite entry?)", r, tok, vocab_size));
        if (stop.count(tok)) g.finish_reason = "stop";
        else {
            g.tokens.push_back(tok);
            if ((int)g.tokens.size() >= opt.max_new_tokens) g.finish_reason = "length";
            else if ((int)prompts[r].size() + (int)g.tokens.size() - 1 >= max_context) g.finish_reason = "context";
        }
        return g.finish_reason.empty();
    };

    for (size_t first = 0; first < prompts.size(); first += (size_t)max_batch) {
        std::vector<int> batch;
        for (size_t r = first; r < std::min(prompts.size(), first + (size_t)max_batch); ++r) batch.push_back((int)r);
        std::map<int, int> slot_of;
        LoopHooks::Rows dec;
        bool have_dec = false;
        auto cleanup = [&]() {
            if (have_dec && dec.close) {
                have_dec = false;
                dec.close();
            }
            for (auto& kv : slot_of) hooks.free_slot(kv.second);        // an error in the middle gives the slots back too
            slot_of.clear();
        };
        try {
            for (int r : batch) slot_of[r] = hooks.alloc_slot();
            std::vector<int> live = batch;
            auto settle_all = [&](const std::vector<int>& who, const std::vector<int>& drawn) {
                if (opt.on_step) opt.on_step(who, drawn);
                std::vector<int> next;
                for (size_t i = 0; i < who.size(); ++i) {
                    if (settle(who[i], drawn[i])) next.push_back(who[i]);
                    else {
                        hooks.free_slot(slot_of[who[i]]);
                        slot_of.erase(who[i]);
                    }
                }
                return next;
            };
            {
                std::vector<int> slots;
                std::vector<std::vector<int>> toks, want;
                std::vector<int> zeros(live.size(), 0);
                for (int r : live) {
                    slots.push_back(slot_of[r]);
                    toks.push_back(prompts[r]);
                    want.push_back({(int)prompts[r].size() - 1});
                }
                hooks.step(slots, toks, want);
                live = settle_all(live, hooks.sample(live, zeros));
            }
            if (hooks.decoder && !live.empty()) {
                const std::vector<int> rows = live;        // row i of the decoder belongs to request rows[i], for good
                std::vector<int> slots, firsts, done;
                for (int r : rows) {
                    slots.push_back(slot_of[r]);
                    firsts.push_back(results[r].tokens.back());
                    done.push_back((int)results[r].tokens.size());
                }
                dec = hooks.decoder(slots, firsts, rows, done);
                have_dec = true;
                while (!live.empty()) {
                    std::vector<int> feed;
                    for (int r : rows) feed.push_back(slot_of.count(r) ? results[r].tokens.back() : 0);
                    const std::vector<int> drawn_rows = dec.step(feed);
                    std::vector<int> drawn;
                    for (int r : live) drawn.push_back(drawn_rows[std::find(rows.begin(), rows.end(), r) - rows.begin()]);
                    if (opt.on_step) opt.on_step(live, drawn);
                    std::vector<int> next;
                    for (size_t i = 0; i < live.size(); ++i) {
                        const int r = live[i];
                        if (settle(r, drawn[i])) next.push_back(r);
                        else {
                            dec.retire((int)(std::find(rows.begin(), rows.end(), r) - rows.begin()));
                            hooks.free_slot(slot_of[r]);
                            slot_of.erase(r);
                        }
                    }
                    live = next;
                }
            }
            while (!live.empty()) {
                std::vector<int> slots, steps;
                std::vector<std::vector<int>> toks, want;
                for (int r : live) {
                    slots.push_back(slot_of[r]);
                    toks.push_back({results[r].tokens.back()});
                    want.push_back({0});
                    steps.push_back((int)results[r].tokens.size());
                }
                hooks.step(slots, toks, want);
                live = settle_all(live, hooks.sample(live, steps));
            }
        } catch (...) {
            try { cleanup(); } catch (...) {}
            throw;
        }
        cleanup();
    }
    return results;
}

}  // namespace friday
