"""Choosing the next token of every sequence from its row of logits.

temperature 0 is greedy: the first maximum wins and NaN/Inf are skipped, the rule of
the reference's argmaxLogits (main.cpp:90-101), which is all the reference samples
with.  temperature > 0 draws from softmax(logits / temperature); the draw of a sequence
is decided by (seed, the sequence's stream number, how many tokens it has drawn), so it
does not depend on which other sequences share its batch.  The work is done by the
sampling kernel on the device; only the chosen ids come back.
"""
from dataclasses import dataclass

import torch

from .. import ops


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")


class Sampler:
    def __init__(self, params: SamplingParams, device):
        self.params = params
        self.device = device

    def sample_device(self, logits, streams, steps):
        """logits [n, vocab] fp32 on the device -> int32 [n] on the device."""
        n = logits.shape[0]
        meta = torch.tensor([list(streams), list(steps)], dtype=torch.int32).to(self.device, non_blocking=True)
        temp = torch.full((n,), float(self.params.temperature), dtype=torch.float32, device=self.device)
        return ops.sample(logits, temp, meta[0], meta[1], self.params.seed)

    def sample(self, logits, streams, steps):
        """The chosen token of every row, as a list of ints on the host."""
        return [int(t) for t in self.sample_device(logits, streams, steps).cpu().tolist()]
