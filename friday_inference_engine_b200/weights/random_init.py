"""Random weights from a seed: a tensor source for the loader, and a writer of model
folders (config.json + model.safetensors).

Every tensor has a stream of its own, derived from (seed, tensor name), so any tensor
can be made alone, in any order, and a model folder written from a seed always holds
the same numbers.  Matrices, tables and biases are N(0, 0.02); norm weights are
1 + N(0, 0.02).  Numbers are drawn in fp32 and rounded once to the storage dtype.
The reference has no such mode (its tests draw N(0,1) fp16 tensors per kernel:
tests/kernels/test_decode_attention.cu:45-50).
"""
import hashlib
import json
import os

import torch

from .safetensors_io import write_safetensors

STD = 0.02


def _stream_seed(seed, name):
    h = hashlib.sha256(("%d\0%s" % (int(seed), name)).encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


class RandomSource:
    """Offers the tensors that `expected` (name -> Param) names, drawn from `seed`.

    device "cpu" gives numbers that are the same on every machine (model folders, tests);
    a CUDA device draws there, which is much faster for billions of parameters and is
    what measurements with random weights use.
    """

    def __init__(self, expected, seed, dtype=torch.bfloat16, device="cpu"):
        self.expected = dict(expected)
        self.seed = int(seed)
        self.dtype = dtype
        self.device = torch.device(device)
        self.path = "random weights (seed %d)" % self.seed

    def names(self):
        return list(self.expected)

    def dtype_shape(self, name):
        p = self.expected[name]
        return (torch.int32 if p.kind == "int" else self.dtype), p.shape

    def tensor(self, name):
        p = self.expected[name]
        gen = torch.Generator(device=self.device)
        gen.manual_seed(_stream_seed(self.seed, name))
        if p.kind == "int":
            return torch.zeros(p.shape, dtype=torch.int32, device=self.device)
        t = torch.randn(p.shape, generator=gen, dtype=torch.float32, device=self.device) * STD
        if p.init == "one":
            t = t + 1.0
        return t.to(self.dtype)


def expected_params(model):
    out = {}
    for name, _, _, param in model.named_params():
        out.setdefault(name, param)
    return out


def write_model_dir(path, config_dict, expected, seed, dtype=torch.bfloat16):
    """Writes config.json and model.safetensors for `expected` (name -> Param)."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(config_dict, f, indent=1, sort_keys=True)
    src = RandomSource(expected, seed, dtype=dtype, device="cpu")
    write_safetensors(os.path.join(path, "model.safetensors"), {n: src.tensor(n) for n in src.names()},
                      metadata={"format": "pt", "seed": seed})
    return path
