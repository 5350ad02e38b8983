"""Decoding one token per sequence, step after step, with everything the kernels read in
buffers that keep their addresses, so that the step can be captured once in a CUDA graph
and replayed (the reference captures its layer stack the same way and lets kernels read
the position from device memory: transformer.cpp:1465-1483, attention_kernels.cu:33).

A step is: embedding of each row's token, the model's program over the cache, final norm
and head for every row, the sampler, and `advance` (the chosen token becomes the row's
next input; position and length grow by one).  Between steps the host only reserves cache
pages (a table row changes every 64 tokens) and, if the caller drives the tokens itself
(generation with stop tokens, replayed traces), writes the step's tokens.

It uses the same model, cache, kernels and page tables as the step function; only the
buffers are long-lived.  A row whose sequence has ended is marked dead (row_seq < 0):
kernels skip it and the sampler returns 0 for it.
"""
import gc

import numpy as np
import torch

from .. import ops
from ..cache import PAGE
from ..ops import lib
from .step import StepContext


class DeviceDecoder:
    def __init__(self, engine, slots, first_tokens, temperature=0.0, seed=0, streams=None, steps_done=None,
                 use_graph=True):
        self.engine = engine
        self.cache, self.model, self.device = engine.cache, engine.model, engine.device
        self.slots = list(slots)
        self.live = [True] * len(self.slots)
        n = len(self.slots)
        self.n = n
        dev = self.device
        i32 = dict(dtype=torch.int32, device=dev)
        self.tokens = torch.tensor(list(first_tokens), **i32)
        self.row_seq = torch.arange(n, **i32)
        self.row_pos = torch.tensor([self.cache.lens[s] for s in self.slots], **i32)
        self.kv_len = self.row_pos + 1
        self.sampled = torch.zeros(n, **i32)
        self.temperature = torch.full((n,), float(temperature), dtype=torch.float32, device=dev)
        self.streams = torch.tensor(list(streams) if streams is not None else list(range(n)), **i32)
        self.draws = torch.tensor(list(steps_done) if steps_done is not None else [0] * n, **i32)
        self.seed = int(seed)
        self.tables_host = self.cache.tables_for(self.slots)
        self.tables = [torch.from_numpy(t.copy()).to(dev) for t in self.tables_host]
        # Launch shapes depend on how long the longest sequence may be (how many ways its keys are split), so a
        # captured step serves lengths up to a bound; when a sequence outgrows it, the next bound's step is
        # captured.  Bounds double from 1,024 tokens.
        self.bound = self._bound_for(max(self.cache.lens[s] for s in self.slots) + 1)
        self.ctx = StepContext(self, self.slots, [1] * n, [self.bound] * n)
        self.ctx.tokens, self.ctx.row_seq, self.ctx.row_pos = self.tokens, self.row_seq, self.row_pos
        self.ctx.seq_start = torch.arange(n, **i32)              # one row per sequence
        self.ctx.seq_qlen = torch.ones(n, **i32)
        self.ctx.seq_pos0 = self.row_pos                          # the row's position is the sequence's
        self.ctx.tables = self.tables
        self.ctx.seq_slots = torch.as_tensor(self.slots, dtype=torch.int64, device=dev) if self.cache.states else None
        self._scratch = None
        self._pinned = torch.empty((n,), dtype=torch.int32).pin_memory() if dev.type == "cuda" else None
        self._pinned_out = torch.empty((n,), dtype=torch.int32).pin_memory() if dev.type == "cuda" else None
        self._copied = None           # event after the last copy out of _pinned
        self.use_graph = bool(use_graph) and dev.type == "cuda"
        self.graph = None
        self.graphs = {}              # bound -> captured step
        self.eager_steps = 0
        self.launches_per_step = 0
        self.logits = None
        # All layers of the step in one persistent kernel, where the model and the batch allow it.
        from . import fused_decode
        self.fused = fused_decode.FusedLayers(self) if fused_decode.applicable(self.model, self.cache, n) else None

    def reset(self, slots, first_tokens, temperature=0.0, seed=0, streams=None, steps_done=None):
        """Takes over another batch of the same size: the buffers keep their addresses, so the captured steps
        stay valid (they are captured again only if the sampler's seed changes, which is a kernel argument, or
        if a mixer keeps state that it addresses from the host)."""
        n = self.n
        assert len(slots) == n
        self.slots[:] = list(slots)
        self.ctx.slots[:] = self.slots
        self.live = [True] * n
        i32 = dict(dtype=torch.int32)
        self.tokens.copy_(torch.tensor(list(first_tokens), **i32))
        self.row_seq.copy_(torch.arange(n, **i32))
        self.row_pos.copy_(torch.tensor([self.cache.lens[s] for s in self.slots], **i32))
        self.kv_len.copy_(self.row_pos + 1)
        self.temperature.fill_(float(temperature))
        self.streams.copy_(torch.tensor(list(streams) if streams is not None else list(range(n)), **i32))
        self.draws.copy_(torch.tensor(list(steps_done) if steps_done is not None else [0] * n, **i32))
        if int(seed) != self.seed or self.cache.states:
            self.seed = int(seed)
            self.graphs.clear()
        if self.ctx.seq_slots is not None:
            self.ctx.seq_slots.copy_(torch.as_tensor(self.slots, dtype=torch.int64))
        fresh = self.cache.tables_for(self.slots)
        for t_host, t_dev, t_new in zip(self.tables_host, self.tables, fresh):
            t_host[:] = t_new
            t_dev.copy_(torch.from_numpy(t_new))
        self.bound = self._bound_for(max(self.cache.lens[s] for s in self.slots) + 1)
        self.ctx.max_kv_len = self.bound
        self.ctx.kv_lens = [self.bound] * n
        self.graph = self.graphs.get(self.bound)
        self._copied = None
        return self

    def _bound_for(self, length):
        bound = 1024
        while bound < length:
            bound *= 2
        return min(bound, max(self.cache.max_seq_tokens, 1))

    # what parts ask of a context
    def scratch(self, n_floats, device):
        if self._scratch is None or self._scratch.numel() < n_floats:
            self.graphs.clear()       # captured steps point at the old buffer: they are captured again when needed
            self.graph = None
            self._scratch = torch.empty((int(n_floats),), dtype=torch.float32, device=device)
        return self._scratch

    def _views(self):
        return [None if call.cache is None
                else self.cache.view(call.cache, call.write, self.tables, self.ctx.seq_slots, self.slots)
                for call in self.model.program]

    def _body(self):
        if self.fused is not None:
            ops.embedding(self.tokens, self.model.embedding, out=self.fused.x)
            x, normed = self.fused.run(self.row_seq, self.row_pos, self.bound), None
        else:
            x, normed = self.model.run(self.tokens, self.ctx, self._views(), final_norm=True)
        self.logits = self.model.logits(x, normed=normed)
        ops.sample(self.logits, self.temperature, self.streams, self.draws, self.seed, row_live=self.row_seq,
                   out=self.sampled)
        ops.advance(self.tokens, self.sampled, self.row_pos, self.kv_len, self.row_seq, self.draws)

    def _sync_tables(self):
        slots = [s for s, alive in zip(self.slots, self.live) if alive]
        if not any(self.cache.lens[s] % PAGE == 0 for s in slots):
            return                                       # nobody crosses into a new page: tables stand
        self.cache.reserve(slots, [1] * len(slots))
        for t_host, t_dev, fresh in zip(self.tables_host, self.tables, self.cache.tables_for(self.slots)):
            for i, alive in enumerate(self.live):
                if not alive:
                    fresh[i] = t_host[i]                 # a dead row keeps its stale table; nothing reads it
            if not np.array_equal(t_host, fresh):
                t_host[:] = fresh
                t_dev.copy_(torch.from_numpy(fresh), non_blocking=False)

    def step(self, tokens=None):
        """One decode step.  tokens: host list with each row's input token (dead rows: anything), or None to go
        on with the tokens that the previous step chose.  The chosen tokens are in self.sampled afterwards."""
        self._sync_tables()
        need = self._bound_for(max([self.cache.lens[s] for s, alive in zip(self.slots, self.live) if alive] or [0]) + 1)
        if need != self.bound:
            self.bound = need
            self.ctx.max_kv_len = need
            self.ctx.kv_lens = [need] * self.n
            self.graph = self.graphs.get(need)
        if tokens is not None:
            if self._pinned is not None:
                if self._copied is not None:
                    self._copied.synchronize()          # the copy of the step before has read the buffer
                self._pinned.numpy()[:] = np.asarray(tokens, dtype=np.int32)
                self.tokens.copy_(self._pinned, non_blocking=True)
                self._copied = torch.cuda.Event()
                self._copied.record()
            else:
                self.tokens.copy_(torch.tensor(list(tokens), dtype=torch.int32))
        if not self.use_graph:
            self._body()
        elif self.graph is None and self.eager_steps < 1:
            before = lib.launch_count()
            self._body()                                  # builds libraries, sizes scratch, warms allocations
            self.launches_per_step = lib.launch_count() - before
            self.eager_steps += 1
        else:
            if self.graph is None:
                self.graph = torch.cuda.CUDAGraph()
                torch.cuda.synchronize()
                before = lib.launch_count()
                # Captured steps of decoders that nothing refers to any more must not be destroyed while this one
                # is being captured (the runtime refuses that and the capture is lost): collect them now, and keep
                # the collector quiet until the capture has ended.
                gc.collect()
                collecting = gc.isenabled()
                gc.disable()
                try:
                    with torch.cuda.graph(self.graph):
                        self._body()
                finally:
                    if collecting:
                        gc.enable()
                lib.add_launches(before - lib.launch_count())     # capturing launched nothing
                self.graphs[self.bound] = self.graph
            self.graph.replay()
            lib.add_launches(self.launches_per_step)
        live_slots = [s for s, alive in zip(self.slots, self.live) if alive]
        self.cache.commit(live_slots, [1] * len(live_slots))

    def check(self):
        if self.fused is not None:
            self.fused.check()

    def read_sampled(self):
        """The tokens that the last step chose, as a host list (waits for the step)."""
        if self._pinned_out is not None:
            self._pinned_out.copy_(self.sampled, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return self._pinned_out.tolist()
        return self.sampled.tolist()

    def retire(self, index):
        """Row `index` has ended: kernels skip it from now on.  The caller frees its slot."""
        self.live[index] = False
        self.row_seq[index] = -1

    def close(self):
        """Hands the decoder back to the engine, which keeps it (buffers, captured steps) for the next batch of
        this size."""
        self.engine.keep_decoder(self)
