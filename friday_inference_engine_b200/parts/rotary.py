"""Rotary position encoding, NeoX pairing: the pair (i, i + rotary_dim/2) of every
query and key head is rotated by the angle pos / theta^(2i / rotary_dim).

The angle is formed as the reference forms it (cuda_math_kernels.cu:337-339,
cpu_ops.cpp:26-30): the denominator theta^(2i/d) in fp32, then one fp32 division of
the position by it.  The denominators are a table of rotary_dim/2 numbers, made once
here; the kernel divides and takes sine and cosine per row.
"""
import numpy as np
import torch

from .base import Part, register_part


@register_part("position", "rotary_neox")
class RotaryNeox(Part):
    category = "position"
    rotary = True

    def __init__(self, env, theta, head_dim, rotary_dim=None):
        super().__init__(env)
        self.theta = float(theta)
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim or head_dim)
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError("rotary_dim %d must be even and at most head_dim %d" % (self.rotary_dim, self.head_dim))
        i = np.arange(self.rotary_dim // 2, dtype=np.float32)
        table = np.power(np.float32(self.theta), (np.float32(2.0) * i) / np.float32(self.rotary_dim))
        self._denom = torch.from_numpy(table.astype(np.float32)).to(env.device)

    def denominators(self):
        return self._denom


@register_part("position", "none")
class NoPosition(Part):
    """Leaves queries and keys as they are."""
    category = "position"
    rotary = True          # handled by the same kernel, with the rotation switched off

    def __init__(self, env, head_dim=0):
        super().__init__(env)
        self.rotary_dim = 0

    def denominators(self):
        return None
