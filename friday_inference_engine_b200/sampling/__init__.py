"""Sampling lives in the library: sampling/sampler.cpp marshals a step's streams and counters,
csrc/sampling.cu chooses (greedy: the first maximum wins; temperature: softmax and an
inverse-CDF draw from a Philox stream keyed by seed, request number and step).  From Python
it is reached through Engine.generate(temperature=..., seed=...) and ops.sample."""
