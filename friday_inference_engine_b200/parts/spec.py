"""The description of a model as data: which parts, with which constants, in which order.

An architecture turns its typed configuration into a ModelSpec; everything below the
architecture (parts, cache, step function, loader) works from the ModelSpec alone and
never asks which model it is in.
"""
from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class PartSpec:
    """One part: `kind` names a registered class of its category, `params` are the sizes
    and constants it is built with, `prefix` is what its tensor names start with inside
    its parent."""
    kind: str
    params: dict = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    layer: index into ModelSpec.layers (a layer may be named by several entries).
    cache: the cache entry that the layer's mixer uses in this call, or None if the mixer
           keeps nothing.  Entries are numbered by the architecture; two calls may name
           the same entry.
    write: False lets the mixer read an entry that another call has filled, without
           writing to it.
    """
    layer: int
    cache: Optional[int] = None
    write: bool = True


@dataclass
class ModelSpec:
    architecture: str
    vocab_size: int
    width: int
    max_positions: int
    embedding: str                 # tensor name of the token table [vocab, width]
    layers: list                   # PartSpec of category "block", one per layer
    program: list                  # LayerCall, in run order
    final_norm: PartSpec
    head: Optional[str]            # tensor name of the head [vocab, width]; None: the token table is the head

    def cache_entries(self):
        """entry id -> index of the program entry that writes it."""
        owners = {}
        for i, call in enumerate(self.program):
            if call.cache is None:
                continue
            if call.write:
                if call.cache in owners:
                    raise ValueError("cache entry %d is written by program entries %d and %d"
                                     % (call.cache, owners[call.cache], i))
                owners[call.cache] = i
        for i, call in enumerate(self.program):
            if call.cache is not None and not call.write:
                if call.cache not in owners or owners[call.cache] > i:
                    raise ValueError("program entry %d reads cache entry %d before anything wrote it"
                                     % (i, call.cache))
        return owners
