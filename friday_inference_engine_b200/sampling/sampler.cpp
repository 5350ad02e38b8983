// Sampler (sampling.h): marshals a step's streams and counters to the device and runs the sampling kernel.
#include "friday/sampling.h"

namespace friday {

Sampler::Sampler(Ops& ops, const SamplingParams& params) : ops_(ops), params_(params), arena_(ops.stream(), 1 << 16) {
    if (params.temperature < 0) throw GenerationError("temperature must not be negative");
}

std::vector<int> Sampler::sample(const Tensor& logits, const std::vector<int>& streams, const std::vector<int>& steps) {
    const size_t n = streams.size();
    if ((size_t)logits.rows() != n || steps.size() != n)
        throw GenerationError("the sampler needs one stream and one step count per row of logits");
    arena_.reset();
    std::vector<int> host(2 * n);
    std::vector<float> temp(n, params_.temperature);
    for (size_t i = 0; i < n; ++i) {
        host[i] = streams[i];
        host[n + i] = steps[i];
    }
    int* dev = (int*)arena_.alloc(3 * n * sizeof(int));
    float* dtemp = (float*)arena_.alloc(n * sizeof(float));
    cudaStream_t s = ops_.stream();
    cuda_check(cudaMemcpyAsync(dev, host.data(), 2 * n * sizeof(int), cudaMemcpyHostToDevice, s), "cudaMemcpyAsync");
    cuda_check(cudaMemcpyAsync(dtemp, temp.data(), n * sizeof(float), cudaMemcpyHostToDevice, s), "cudaMemcpyAsync");
    ops_.sample(logits, dtemp, dev, dev + n, params_.seed, nullptr, dev + 2 * n);
    std::vector<int> ids(n);
    cuda_check(cudaMemcpyAsync(ids.data(), dev + 2 * n, n * sizeof(int), cudaMemcpyDeviceToHost, s), "cudaMemcpyAsync");
    cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");      // also makes the pageable copies above safe to free
    return ids;
}

}  // namespace friday
