// Runs the reference's own engine (friday::Engine, CPU backend) on a GGUF file and prints the logits of
// every position: one line per token, space-separated floats.  Links against the reference's
// libfriday_engine.a, built from its unmodified sources; see make_golden.py.
//   reference_driver model.gguf ctx tok0 tok1 ...
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "engine.h"

int main(int argc, char** argv) {
    if (argc < 4) return 2;
    friday::EngineOptions opt;
    opt.model_path = argv[1];
    opt.max_ctx = std::atoi(argv[2]);
    opt.backend = friday::BackendKind::Cpu;
    opt.cpu_threads = 1;
    friday::Engine engine(opt);
    std::vector<float> logits(engine.vocabSize());
    for (int i = 3; i < argc; ++i) {
        engine.step(std::atoi(argv[i]), i - 3, logits.data());
        for (size_t v = 0; v < logits.size(); ++v) std::printf("%s%.9g", v ? " " : "", logits[v]);
        std::printf("\n");
    }
    return 0;
}
