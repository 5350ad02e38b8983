"""A decoder put together from a ModelSpec: token table, blocks, final norm, head.

It knows nothing of any architecture: the specification says which parts there are and
in which order they run.  `run` takes the tokens of one pass as rows, sends them through
the program, and returns the residual stream; `logits` applies the final norm and the
head to chosen rows only (the reference does this for one row: transformer.cpp:1077-1113).
"""
import torch

from .. import ops
from ..parts.base import BuildEnv, Param, build_part


class DecoderModel:
    def __init__(self, spec, dtype, device):
        self.spec = spec
        self.env = BuildEnv(width=spec.width, dtype=dtype, device=device)
        self.layers = [build_part("block", ls, self.env) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, self.env)
        self.program = list(spec.program)
        self.owners = spec.cache_entries()
        for i, call in enumerate(self.program):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError("program entry %d names layer %d of %d" % (i, call.layer, len(self.layers)))
        self.embedding = None
        self.head = None

    # -- what the loader needs ---------------------------------------------
    def named_params(self):
        s = self.spec
        yield s.embedding, self, "embedding", Param((s.vocab_size, s.width))
        for ls, layer in zip(s.layers, self.layers):
            yield from layer.named_params(ls.prefix)
        yield from self.final_norm.named_params(s.final_norm.prefix)
        if s.head is not None:
            yield s.head, self, "head", Param((s.vocab_size, s.width))

    def ignorable_tensors(self):
        """A checkpoint whose head is tied to the token table may still carry a copy of it."""
        return ("lm_head.weight",) if self.spec.head is None else ()

    def set_tensor(self, name, tensor):
        setattr(self, name, tensor)

    def finalize(self):
        for layer in self.layers:
            layer.finalize()
        self.final_norm.finalize()
        if self.spec.head is None:
            self.head = self.embedding           # one copy in memory

    def cache_requests(self):
        """cache entry -> what the mixer of the call that writes it asks for."""
        return {entry: self.layers[self.program[i].layer].cache_request() for entry, i in self.owners.items()}

    # -- the forward pass of one pass of the step function -------------------
    def run(self, tokens, ctx, views, final_norm=False):
        """tokens: int32 [rows] on the device; views: one cache view (or None) per program entry.  Returns the
        residual stream, and with final_norm also its final norm (every row's), as `logits` takes it.

        A block that chains norms is told which norm follows it (the next block's first, or the final one), so
        that its last product can begin that norm, and is handed its own first norm if the block before did so."""
        x = ops.embedding(tokens, self.embedding)
        normed = None
        for i, (call, view) in enumerate(zip(self.program, views)):
            block = self.layers[call.layer]
            if not block.chains_norm:
                x, normed = block.forward(x, ctx, view), None
                continue
            if i + 1 < len(self.program):
                nxt = self.layers[self.program[i + 1].layer]
                then = nxt.first_norm if nxt.chains_norm else None
            else:
                then = self.final_norm if final_norm else None
            x, normed = block.forward(x, ctx, view, normed=normed, then=then)
        return (x, normed) if final_norm else x

    def logits(self, x, rows=None, normed=None):
        """fp32 logits [n, vocab] of the rows `rows` (int32 device tensor) of x, or of all rows.  normed: the
        final norm of all rows of x, if the caller has it."""
        if rows is not None:
            x, normed = ops.gather_rows(rows, x), None
        if normed is None:
            normed = self.final_norm.forward(x)
        return ops.linear(normed, self.head, out_dtype=torch.float32)

    def parameter_bytes(self):
        seen, total = set(), 0

        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()

        def walk(part):
            for v in vars(part).values():
                if hasattr(v, "data_ptr"):
                    add(v)
            for v in part.tensors.values():
                add(v)
            for _, child in part.children:
                walk(child)

        add(self.embedding)
        add(self.head)
        for layer in self.layers:
            walk(layer)
        walk(self.final_norm)
        return total
