// A C++ program over the library's public interface (include/friday/engine.h): loads a model folder, generates
// greedy tokens for the prompts on standard input (one line of token ids each), and prints them; then feeds the first
// prompt through the single-sequence conveniences prefill() and step() and prints the argmax of each row of logits.
//   generate_main MODEL_DIR DTYPE MAX_NEW_TOKENS < prompts.txt
#include <cstdio>
#include <iostream>
#include <sstream>

#include "friday/engine.h"

int main(int argc, char** argv) {
    if (argc < 4) return 2;
    try {
        friday::EngineOptions opt;
        opt.model_path = argv[1];
        opt.dtype = argv[2];
        opt.max_ctx = 128;
        opt.max_batch = 2;
        friday::Engine engine(opt);
        std::vector<std::vector<int>> prompts;
        for (std::string line; std::getline(std::cin, line);) {
            std::istringstream in(line);
            std::vector<int> p;
            for (int t; in >> t;) p.push_back(t);
            if (!p.empty()) prompts.push_back(p);
        }
        friday::GenerateOptions gen;
        gen.max_new_tokens = atoi(argv[3]);
        for (const friday::Generation& g : engine.generate(prompts, gen)) {
            for (int t : g.tokens) printf("%d ", t);
            printf("[%s]\n", g.finish_reason.c_str());
        }
        std::vector<float> logits((size_t)engine.vocabSize());
        auto argmax = [&]() {
            int best = 0;
            for (int i = 1; i < engine.vocabSize(); ++i)
                if (logits[i] > logits[best]) best = i;
            return best;
        };
        const std::vector<int>& p = prompts[0];
        engine.prefill(p.data(), (int)p.size() - 1, 0, logits.data());
        printf("prefill %d\n", argmax());
        engine.step(p.back(), (int)p.size() - 1, logits.data());
        printf("step %d\n", argmax());
        fprintf(stderr, "%s\n", engine.summary().c_str());
    } catch (const std::exception& e) {
        fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
    return 0;
}
