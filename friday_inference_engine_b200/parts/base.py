"""What every part is, and the registry that the configuration chooses parts from.

Categories and the interface each must offer:

  norm           forward(x[rows, width]) -> tensor of the same shape
  position       rotary parts: denominators() -> fp32 tensor [rotary_dim/2] and rotary_dim;
                 the mixer hands them to the kernel that rotates q and k.  A position part
                 that is not rotary offers apply(qkv, ctx, n_heads, n_kv_heads, head_dim).
  mixer          cache_request() -> KVRequest | StateRequest | None
                 forward(h, residual, ctx, cache) -> residual + mix(h)      [rows, width]
  feed_forward   forward(h, residual, ctx) -> residual + f(h)               [rows, width]
  block          cache_request() (its mixer's), forward(x, ctx, cache) -> x

Optional, for parts that end in a product: a mixer, feed-forward or block whose class sets
`chains_norm = True` takes `then=` (the norm part that will be applied to its result, or
None) and returns the pair (result, normed result or None); its input `h` may then be an
`ops.DeferredNorm`, which products accept as it is and `ops.materialize` turns into a
tensor.  A norm part that is a plain RMSNorm says so with `as_rmsnorm() -> (weight, eps)`,
so that the product before it can begin it (ops.linear_norm).  A chaining block also takes
`normed=` (its first norm already applied by the block before) and offers `first_norm`.
Parts that do none of this are called with the plain interface above.

`ctx` is the step's geometry (engine/step.py, StepContext): rows, n_seqs, row_seq and
row_pos (int32 device tensors: the sequence of the step and the position of every row),
seq_slots, q_lens, kv_lens, max_q_len, max_kv_len, and scratch(n_floats).  `cache` is
what the cache hands out for the call's entry: a KVView (pools, this step's block
table, page size, write flag) or a StateView (a tensor [slots, *shape] and the slot of
every sequence); None if the mixer asked for nothing.

A part owns its parameters.  It declares them (`params`: local tensor name -> Param) and
its sub-parts (`children`: pairs of local prefix and Part); the loader walks that tree, so a part
never sees a file.  `finalize` runs once after every parameter is set (to fuse matrices,
build tables).  No part may refer to a model or an architecture.
"""
from dataclasses import dataclass
from typing import Optional

import torch

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block")
_registry = {c: {} for c in CATEGORIES}


def register_part(category, kind, cls=None):
    """register_part("mixer", "my_mixer", MyMixer), or as a decorator with cls omitted."""
    if category not in _registry:
        raise KeyError("unknown part category '%s' (have: %s)" % (category, ", ".join(CATEGORIES)))

    def put(c):
        _registry[category][kind] = c
        return c

    return put if cls is None else put(cls)


def build_part(category, spec, env):
    try:
        cls = _registry[category][spec.kind]
    except KeyError:
        raise KeyError("no %s part named '%s' (registered: %s)"
                       % (category, spec.kind, ", ".join(sorted(_registry[category])) or "none")) from None
    part = cls(env=env, **spec.params)
    part.prefix = spec.prefix
    return part


@dataclass(frozen=True)
class BuildEnv:
    """What a part may know of its surroundings: the width of the residual stream, the
    dtype of activations and the device."""
    width: int
    dtype: torch.dtype
    device: torch.device


@dataclass(frozen=True)
class Param:
    shape: tuple
    kind: str = "float"     # "float": kept in the activation dtype unless stored in 32-bit; "int": int32
    init: str = "normal"    # random-weights mode: "normal" N(0, 0.02); "one": 1 + N(0, 0.02) (norm weights)


@dataclass(frozen=True)
class KVRequest:
    """Keys and values for every position (window None) or for the last `window` only."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequest:
    """A tensor of fixed shape per sequence, zero when the sequence starts."""
    shape: tuple
    dtype: torch.dtype = torch.float32


class Part:
    category = None
    prefix = ""
    chains_norm = False

    def as_rmsnorm(self):
        return None

    def __init__(self, env):
        self.env = env
        self.params = {}      # local name -> Param
        self.children = []    # (local prefix, Part)
        self.tensors = {}     # local name -> torch.Tensor, set by the loader

    def declare(self, name, shape, kind="float", init="normal"):
        self.params[name] = Param(tuple(int(s) for s in shape), kind, init)

    def adopt(self, prefix, part):
        self.children.append((prefix, part))
        return part

    def set_tensor(self, name, tensor):
        self.tensors[name] = tensor

    def finalize(self):
        for _, child in self.children:
            child.finalize()

    def named_params(self, prefix=""):
        """(full tensor name, part, local name, Param) for this part and all below it."""
        for name, p in self.params.items():
            yield prefix + name, self, name, p
        for cp, child in self.children:
            yield from child.named_params(prefix + cp)
