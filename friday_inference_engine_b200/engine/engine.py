"""Engine: the public entry point, in the manner of the reference's friday::Engine
(engine.h:19-72): options in, then step / prefill / generate; callers never handle
device memory unless they ask for it.

Where the reference has an option, its name and meaning are kept: `model_path`,
`max_ctx` (tokens one sequence can hold, default 2048: engine.h:22).  Its options for
CPU offload, a VRAM limit and quantized KV (`vram_gb`, `cpu_threads`, `backend`,
`kv_cache`) have nothing to act on here and are not offered.  New ones: `dtype`,
`max_batch` (sequences alive at once), `max_tokens` (cache capacity), and a
random-weights mode from a configuration and a seed.
"""
import os
from dataclasses import dataclass
from typing import Optional

import torch

from .. import architectures  # noqa: F401  (registers the shipped architectures)
from ..cache import PAGE, Cache
from ..registry import read_config
from ..sampling import Sampler, SamplingParams
from ..weights import RandomSource, SafetensorsFile, expected_params, load_weights
from . import generate as _generate
from .model import DecoderModel
from .step import Stepper

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


def parse_dtype(name):
    if isinstance(name, torch.dtype):
        if name in (torch.bfloat16, torch.float32):
            return name
    elif name in _DTYPES:
        return _DTYPES[name]
    raise ValueError("dtype must be bfloat16 or float32, got %r" % (name,))


@dataclass
class EngineOptions:
    model_path: Optional[str] = None       # folder with config.json and model.safetensors
    config: Optional[dict] = None          # instead of model_path: config.json's content, random weights
    seed: int = 0                          # of the random weights
    dtype: str = "bfloat16"                # "bfloat16": what serving uses; "float32": everything in true 32-bit
    max_ctx: int = 2048                    # tokens one sequence can hold
    max_batch: int = 8                     # sequences alive at once
    max_tokens: Optional[int] = None       # cache capacity in tokens; default max_batch * max_ctx (in pages)
    device: str = "cuda:0"
    prefill_chunk: int = 2048              # tokens of one sequence per pass
    cuda_graphs: bool = True               # decode steps of generate() are captured once and replayed
    random_on_device: bool = True          # random weights are drawn on the device (fast); False: on the CPU


class Engine:
    def __init__(self, options: Optional[EngineOptions] = None, **kw):
        opt = options or EngineOptions(**kw)
        if options is not None and kw:
            raise TypeError("give EngineOptions or keyword options, not both")
        self.options = opt
        self.dtype = parse_dtype(opt.dtype)
        self.device = torch.device(opt.device)
        if (opt.model_path is None) == (opt.config is None):
            raise ValueError("give either model_path (a model folder) or config (random weights)")
        self.arch, self.config = read_config(opt.model_path if opt.model_path is not None else opt.config)
        spec = self.arch.build_spec(self.config)
        self.model = DecoderModel(spec, self.dtype, self.device)
        if opt.model_path is not None:
            path = os.path.join(opt.model_path, "model.safetensors")
            if not os.path.exists(path):
                raise FileNotFoundError("%s: no model.safetensors in the model folder" % opt.model_path)
            source = SafetensorsFile(path)
        else:
            dev = self.device if (opt.random_on_device and self.device.type == "cuda") else "cpu"
            source = RandomSource(expected_params(self.model), opt.seed, dtype=torch.bfloat16, device=dev)
        load_weights(self.model, source)
        if hasattr(source, "close"):
            source.close()
        self.max_ctx = min(int(opt.max_ctx), spec.max_positions)
        self.max_batch = int(opt.max_batch)
        per_seq = (self.max_ctx + PAGE - 1) // PAGE * PAGE
        max_tokens = int(opt.max_tokens) if opt.max_tokens else self.max_batch * per_seq
        self.cache = Cache(self.model.cache_requests(), max_tokens, self.max_ctx, self.dtype, self.device,
                           max_slots=self.max_batch)
        self.stepper = Stepper(self.model, self.cache, chunk=opt.prefill_chunk)
        self._single = None     # slot of the single-sequence conveniences
        self._decoders = {}     # batch size -> a decoder that is not in use (buffers and captured steps kept)

    # -- facts -------------------------------------------------------------
    @property
    def vocab_size(self):
        return self.model.spec.vocab_size

    @property
    def max_context(self):
        return self.max_ctx

    def summary(self):
        s = self.model.spec
        return ("%s on %s, %s: %d layers, width %d, vocabulary %d; weights %.2f GB; cache %.2f GB for %d tokens, "
                "%d sequences of up to %d"
                % (s.architecture, self.device, str(self.dtype).replace("torch.", ""), len(s.layers), s.width,
                   s.vocab_size, self.model.parameter_bytes() / 1e9, self.cache.bytes() / 1e9,
                   self.cache.groups[0].n_pages * PAGE if self.cache.groups else 0, self.max_batch, self.max_ctx))

    # -- the step function ---------------------------------------------------
    def alloc_slot(self):
        return self.cache.alloc_slot()

    def free_slot(self, slot):
        self.cache.free_slot(slot)

    def step(self, slots, tokens, want):
        """Runs `tokens[i]` as the next tokens of the sequence in `slots[i]`, all as one batch,
        and returns fp32 logits [sum(len(w)), vocab] (device tensor) for the places `want[i]`."""
        return self.stepper.step(list(slots), [list(t) for t in tokens], [list(w) for w in want])

    # -- single-sequence conveniences with the reference's meaning (engine.h:44-54) -------
    def _single_at(self, pos):
        if pos == 0:
            if self._single is not None:
                self.cache.free_slot(self._single)
            self._single = self.cache.alloc_slot()
        if self._single is None or self.cache.lens[self._single] != pos:
            raise ValueError("positions must be fed in order, starting at 0 for a new sequence (at %d, got %d)"
                             % (0 if self._single is None else self.cache.lens[self._single], pos))
        return self._single

    def step_token(self, token, pos):
        """One token at position `pos`; returns its logits as a host fp32 tensor [vocab]."""
        out = self.step([self._single_at(pos)], [[int(token)]], [[0]])[0].cpu()
        self.check()
        return out

    def prefill(self, tokens, pos=0):
        """tokens at positions pos .. pos+n-1; returns the logits of the last one (host)."""
        tokens = [int(t) for t in tokens]
        out = self.step([self._single_at(pos)], [tokens], [[len(tokens) - 1]])[0].cpu()
        self.check()
        return out

    # -- generation ------------------------------------------------------------
    def generate(self, prompts, max_new_tokens=100, temperature=0.0, seed=0, stop_token_ids=(), ignore_eos=False,
                 on_step=None):
        """prompts: lists of token ids.  Returns one Generation (tokens, finish_reason) per prompt."""
        sampler = Sampler(SamplingParams(float(temperature), int(seed)), self.device)

        class Rows:
            """The decoder behind the loop's interface: tokens in from the host, chosen ids out to the host."""

            def __init__(rows, slots, first_tokens, streams, steps_done):
                rows.dec = self.decoder(slots, first_tokens, temperature=temperature, seed=seed, streams=streams,
                                        steps_done=steps_done)

            def step(rows, tokens):
                rows.dec.step(tokens)
                return rows.dec.read_sampled()

            def retire(rows, index):
                rows.dec.retire(index)

            def close(rows):
                rows.dec.check()
                rows.dec.close()

        out = _generate.generate(
            prompts, step=self.step, sample=sampler.sample, alloc_slot=self.alloc_slot, free_slot=self.free_slot,
            max_batch=self.max_batch, max_context=self.max_ctx, vocab_size=self.vocab_size,
            max_new_tokens=max_new_tokens, stop_token_ids=stop_token_ids, ignore_eos=ignore_eos, on_step=on_step,
            decoder=Rows)
        self.check()
        return out

    def check(self):
        """Raises if a kernel reported that it gave up on a wait (its results would be invalid)."""
        from .. import ops
        be = ops.backend()
        if hasattr(be, "check_status"):
            be.check_status()

    def decoder(self, slots, first_tokens, temperature=0.0, seed=0, streams=None, steps_done=None):
        """Decoding of the sequences in `slots`, one token each per step(), from buffers that stay on the
        device (engine/decode.py); the step is captured in a CUDA graph unless cuda_graphs is off."""
        from .decode import DeviceDecoder
        kept = self._decoders.pop(len(slots), None)
        if kept is not None:
            return kept.reset(slots, first_tokens, temperature=temperature, seed=seed, streams=streams,
                              steps_done=steps_done)
        return DeviceDecoder(self, slots, first_tokens, temperature=temperature, seed=seed, streams=streams,
                             steps_done=steps_done, use_graph=self.options.cuda_graphs)

    def keep_decoder(self, decoder):
        self._decoders[decoder.n] = decoder
