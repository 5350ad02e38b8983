// Choosing the next token of every sequence from its row of logits.
//
// temperature 0 is greedy: the first maximum wins and NaN/Inf are skipped, the rule of
// the reference's argmaxLogits (main.cpp:90-101), which is all the reference samples
// with.  temperature > 0 draws from softmax(logits / temperature); the draw of a sequence
// is decided by (seed, the sequence's stream number, how many tokens it has drawn), so it
// does not depend on which other sequences share its batch.  The work is done by the
// sampling kernel on the device (csrc/sampling.cu); only the chosen ids come back.
#pragma once
#include <vector>

#include "friday/ops.h"

namespace friday {

struct SamplingParams {
    float temperature = 0.0f;
    uint64_t seed = 0;
};

class Sampler {
public:
    Sampler(Ops& ops, const SamplingParams& params);
    // One id per row of logits [n, vocab] (fp32, device), on the host; streams and steps: one per row.
    std::vector<int> sample(const Tensor& logits, const std::vector<int>& streams, const std::vector<int>& steps);

private:
    Ops& ops_;
    SamplingParams params_;
    Arena arena_;
};

}  // namespace friday
