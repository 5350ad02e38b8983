from .sampler import Sampler, SamplingParams  # noqa: F401
