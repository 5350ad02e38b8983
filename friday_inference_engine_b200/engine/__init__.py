"""Engine: the Python entry point, a thin layer over friday::Engine of libfriday_engine.so
(include/friday/engine.h), in the manner of the reference's friday::Engine
(engine.h:19-72): options in, then step / prefill / generate.

    from friday_inference_engine_b200 import Engine
    eng = Engine(model_path="/models/qwen2.5-7b", dtype="bfloat16", max_ctx=8192, max_batch=8)
    out = eng.generate([[1, 2, 3], [4, 5]], max_new_tokens=32, temperature=0.8, seed=7, stop_token_ids=[151645])

Nothing of the model runs in Python: configuration, weights, parts, cache, the step
function, the decoder with its CUDA graphs and the generation loop are the library's.
Logits come back as torch tensors on the device (or on the host where a method says so);
torch is used for nothing else here.
"""
import json
from ctypes import byref, c_int, c_int64, c_void_p
from dataclasses import asdict, dataclass, field
from typing import Optional

from .. import native
from ..native import (CacheError, CacheFull, ConfigError, GenerationError, KernelError, StepError,  # noqa: F401
                      WeightsError)


@dataclass
class EngineOptions:
    model_path: Optional[str] = None       # folder with config.json and model.safetensors (or an index and shards)
    config: Optional[dict] = None          # instead of model_path: config.json's content, random weights
    seed: int = 0                          # of the random weights
    dtype: str = "bfloat16"                # "bfloat16": what serving uses; "float32": everything in true 32-bit
    max_ctx: int = 2048                    # tokens one sequence can hold
    max_batch: int = 8                     # sequences alive at once
    max_tokens: Optional[int] = None       # cache capacity in tokens; default max_batch * max_ctx (in pages)
    device: str = "cuda:0"
    prefill_chunk: int = 2560              # most tokens of one sequence per pass
    cuda_graphs: bool = True               # decode steps of generate() are captured once and replayed
    random_on_device: bool = True          # random weights are drawn on the device (fast); False: on the host
    profile: bool = False                  # per-step host time and event-bracketed kernel time (Engine.profile())


@dataclass
class Generation:
    tokens: list = field(default_factory=list)
    finish_reason: str = ""                # "stop" | "length" | "context"


def _device_index(device):
    text = str(device)
    if text == "cuda":
        return 0
    if text.startswith("cuda:"):
        return int(text[5:])
    raise KernelError("device %r: this library runs on CUDA devices only, it has no CPU path" % (device,))


class Decoder:
    """One token per sequence per step, from buffers that stay on the device (friday::Decoder)."""

    def __init__(self, engine, handle, n):
        self.engine, self._h, self.n = engine, handle, n

    def step(self, tokens=None):
        """tokens: each row's input token (dead rows: anything), or None to go on with the tokens that the previous
        step chose."""
        native.call("friday_decoder_step", self._h, None if tokens is None else native.ints(tokens))

    def read_sampled(self):
        out = (c_int * self.n)()
        native.call("friday_decoder_sampled", self._h, out)
        return list(out)

    @property
    def logits(self):
        """The last step's logits [rows, vocab], fp32, as a torch tensor on the engine's device."""
        import torch
        out = torch.empty((self.n, self.engine.vocab_size), dtype=torch.float32, device=self.engine.device)
        torch.cuda.current_stream(out.device).synchronize()
        native.call("friday_decoder_logits", self._h, c_void_p(out.data_ptr()), 1)
        return out

    def retire(self, index):
        native.call("friday_decoder_retire", self._h, int(index))

    def info(self):
        return native.call_json("friday_decoder_info", self._h)

    def check(self):
        self.engine.check()

    def close(self):
        """Hands the decoder back to the engine, which keeps it (buffers, captured steps) for the next batch of
        this size."""
        if self._h is not None:
            native.call("friday_decoder_close", self.engine._h, self._h)
            self._h = None

    def __del__(self):
        if getattr(self, "_h", None) is not None and native._lib is not None:
            native._lib.friday_decoder_free(self._h)
            self._h = None


class Engine:
    def __init__(self, options: Optional[EngineOptions] = None, **kw):
        if options is not None and kw:
            raise TypeError("give EngineOptions or keyword options, not both")
        opt = options or EngineOptions(**kw)
        self.options = opt
        if (opt.model_path is None) == (opt.config is None):
            raise ValueError("give either model_path (a model folder) or config (random weights)")
        d = asdict(opt)
        d["device"] = _device_index(opt.device)
        d["dtype"] = str(opt.dtype).replace("torch.", "")
        d = {k: v for k, v in d.items() if v is not None}
        self._h = c_void_p()
        native.call("friday_engine_new", native.text(json.dumps(d)), byref(self._h))
        info = self.info()
        self.vocab_size = info["vocab_size"]
        self.max_ctx = self.max_context = info["max_context"]
        self.max_batch = info["max_batch"]
        self.config = info["config"]
        self.architecture = info["architecture"]
        self.dtype = info["dtype"]
        self.device = "cuda:%d" % info["device"]
        self._stream = info["stream"]

    def __del__(self):
        if getattr(self, "_h", None) and native is not None and native._lib is not None:
            native._lib.friday_engine_free(self._h)
            self._h = None

    # -- facts -------------------------------------------------------------
    def info(self):
        return native.call_json("friday_engine_info", self._h)

    def summary(self):
        return self.info()["summary"]

    def stats(self):
        """The cache's books (slots and pages held, lengths, tables) and the launch counter."""
        return native.call_json("friday_engine_stats", self._h)

    @property
    def launches(self):
        return self.stats()["launches"]

    @property
    def stream(self):
        """The CUDA stream everything runs on, as a torch stream (to record events around steps)."""
        import torch
        return torch.cuda.ExternalStream(self._stream, device=self.device)

    # -- the step function ---------------------------------------------------
    def alloc_slot(self):
        slot = c_int()
        native.call("friday_engine_alloc_slot", self._h, byref(slot))
        return slot.value

    def free_slot(self, slot):
        native.call("friday_engine_free_slot", self._h, int(slot))

    def slot_length(self, slot):
        n = c_int()
        native.call("friday_engine_slot_length", self._h, int(slot), byref(n))
        return n.value

    def step(self, slots, tokens, want, to="device"):
        """Runs `tokens[i]` as the next tokens of the sequence in `slots[i]`, all as one batch, and returns fp32
        logits [sum(len(w)), vocab] for the places `want[i]`: a torch tensor on the device, or with to="host" a
        numpy array."""
        slots = [int(s) for s in slots]
        n_want = sum(len(w) for w in want)
        t_off, t_val = native.ragged(tokens)
        w_off, w_val = native.ragged(want)
        rows = c_int64()
        if to == "host":
            import numpy as np
            out = np.empty((n_want, self.vocab_size), dtype=np.float32)
            ptr, on_device = out.ctypes.data, 0
        else:
            import torch
            out = torch.empty((n_want, self.vocab_size), dtype=torch.float32, device=self.device)
            torch.cuda.current_stream(out.device).synchronize()
            ptr, on_device = out.data_ptr(), 1
        native.call("friday_engine_step", self._h, len(slots), native.ints(slots), t_off, t_val, w_off, w_val,
                    c_void_p(ptr) if n_want else None, on_device, byref(rows))
        return out

    # -- single-sequence conveniences with the reference's meaning (engine.h:44-54) -------
    def step_token(self, token, pos):
        """One token at position `pos`; returns its logits as a host fp32 tensor [vocab]."""
        import torch
        out = torch.empty((self.vocab_size,), dtype=torch.float32)
        native.call("friday_engine_step_token", self._h, int(token), int(pos), c_void_p(out.data_ptr()))
        return out

    def prefill(self, tokens, pos=0):
        """tokens at positions pos .. pos+n-1; returns the logits of the last one (host)."""
        import torch
        tokens = [int(t) for t in tokens]
        out = torch.empty((self.vocab_size,), dtype=torch.float32)
        native.call("friday_engine_prefill", self._h, native.ints(tokens), len(tokens), int(pos), c_void_p(out.data_ptr()))
        return out

    # -- generation ------------------------------------------------------------
    def generate(self, prompts, max_new_tokens=100, temperature=0.0, seed=0, stop_token_ids=(), ignore_eos=False,
                 on_step=None):
        """prompts: lists of token ids.  Returns one Generation (tokens, finish_reason) per prompt."""
        prompts = [[int(t) for t in p] for p in prompts]
        off, val = native.ragged(prompts)
        opts = {"max_new_tokens": int(max_new_tokens), "temperature": float(temperature), "seed": int(seed),
                "stop_token_ids": [int(t) for t in stop_token_ids], "ignore_eos": bool(ignore_eos)}
        failure = []

        def hook(_user, n, reqs, toks):
            try:
                on_step([reqs[i] for i in range(n)], [toks[i] for i in range(n)])
            except Exception as e:  # noqa: BLE001 - raised again once the library has returned
                failure.append(e)

        cb = native.ON_STEP(hook) if on_step is not None else native.ON_STEP()
        out = native.call_json("friday_engine_generate", self._h, len(prompts), off, val, native.text(json.dumps(opts)),
                               cb, None)
        if failure:
            raise failure[0]
        return [Generation(list(g["tokens"]), g["finish_reason"]) for g in out]

    def set_trace(self, tensor):
        """For measurements: the next tensor.shape[0] tensor-core products fill tensor[launch] ([sm_count, 16] int64)
        with their CTAs' time stamps; None switches it off."""
        if tensor is None:
            native.call("friday_engine_set_trace", self._h, None, 0)
        else:
            native.call("friday_engine_set_trace", self._h, c_void_p(tensor.data_ptr()), int(tensor.shape[0]))

    def check(self):
        """Raises KernelError if a kernel reported that it gave up on a wait (its results would be invalid)."""
        native.call("friday_engine_check", self._h)

    def profile(self):
        """Host time per step and event-bracketed device time per kind of kernel since the last call (needs the
        option profile=True)."""
        return native.call_json("friday_engine_profile", self._h)

    def decoder(self, slots, first_tokens, temperature=0.0, seed=0, streams=None, steps_done=None):
        """Decoding of the sequences in `slots`, one token each per step(), from buffers that stay on the device;
        the step is captured in a CUDA graph unless cuda_graphs is off."""
        slots = [int(s) for s in slots]
        h = c_void_p()
        native.call("friday_decoder_new", self._h, len(slots), native.ints(slots), native.ints(first_tokens),
                    float(temperature), int(seed), None if streams is None else native.ints(streams),
                    None if steps_done is None else native.ints(steps_done), byref(h))
        return Decoder(self, h, len(slots))


def generate_loop(prompts, *, step, sample, alloc_slot, free_slot, max_batch, max_context, vocab_size,
                  max_new_tokens=100, stop_token_ids=(), ignore_eos=False):
    """The library's generation loop alone (engine/generate.cpp), with the step function, the sampler and the slot
    book-keeping handed in as Python callables, so that its decisions can be tested without a model:
    step(slots, tokens, want); sample(streams, steps) -> ids; alloc_slot() -> slot; free_slot(slot).
    An exception raised by a callable ends the loop (slots are given back first) and is raised again here."""
    failure = []

    def guarded(fn):
        def run(*args):
            try:
                return fn(*args)
            except Exception as e:  # noqa: BLE001 - raised again once the library has returned
                failure.append(e)
                return 1
        return run

    @guarded
    def c_step(_user, n, slots, t_off, t_val, w_off, w_val):
        step([slots[i] for i in range(n)], [[t_val[j] for j in range(t_off[i], t_off[i + 1])] for i in range(n)],
             [[w_val[j] for j in range(w_off[i], w_off[i + 1])] for i in range(n)])
        return 0

    @guarded
    def c_sample(_user, n, streams, steps, out):
        ids = sample([streams[i] for i in range(n)], [steps[i] for i in range(n)])
        for i in range(n):
            out[i] = int(ids[i])
        return 0

    @guarded
    def c_alloc(_user, out):
        out[0] = int(alloc_slot())
        return 0

    @guarded
    def c_free(_user, slot):
        free_slot(slot)
        return 0

    hooks = native.LoopHooks(None, native.STEP_HOOK(c_step), native.SAMPLE_HOOK(c_sample), native.ALLOC_HOOK(c_alloc),
                             native.FREE_HOOK(c_free))
    prompts = [[int(t) for t in p] for p in prompts]
    off, val = native.ragged(prompts)
    opts = {"max_new_tokens": int(max_new_tokens), "stop_token_ids": [int(t) for t in stop_token_ids],
            "ignore_eos": bool(ignore_eos)}
    try:
        out = native.call_json("friday_generate_loop", len(prompts), off, val, byref(hooks), int(max_batch),
                               int(max_context), int(vocab_size), native.text(json.dumps(opts)))
    except native.FridayError:
        if failure:
            raise failure[0] from None
        raise
    return [Generation(list(g["tokens"]), g["finish_reason"]) for g in out]
