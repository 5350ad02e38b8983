"""Gated feed-forward: x + Wd (silu(Wg h) * (Wu h)).

Gate and up are one product, as the reference runs the two in one launch
(transformer.cpp:1064-1066): their rows are stacked alternately (gate 0, up 0, gate 1,
...), so that every tile of the product holds both halves of a pair and
silu(z) = z / (1 + e^-z) times up (cpu_ops.cpp:85-101, without its shortcuts for
|z| > 20) can be applied in the product's epilogue; the residual is added in the down
product's epilogue (transformer.cpp:1072).
"""
import torch

from .. import ops
from .base import Part, register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    category = "feed_forward"

    def __init__(self, env, inner):
        super().__init__(env)
        self.inner = int(inner)
        self.declare("gate_proj.weight", (self.inner, env.width))
        self.declare("up_proj.weight", (self.inner, env.width))
        self.declare("down_proj.weight", (env.width, self.inner))

    def finalize(self):
        super().finalize()
        t = self.tensors
        ws = [t.pop("gate_proj.weight"), t.pop("up_proj.weight")]
        wdt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_gate_up = torch.stack([w.to(wdt) for w in ws], dim=1).reshape(2 * self.inner, -1).contiguous()
        self.w_down = t["down_proj.weight"]

    chains_norm = True

    def forward(self, h, residual, ctx, then=None):
        inner = ops.linear_swiglu(h, self.w_gate_up)
        norm = then.as_rmsnorm() if then is not None else None
        if norm is not None:
            return ops.linear_norm(inner, self.w_down, norm[0], norm[1], residual=residual)
        return ops.linear(inner, self.w_down, residual=residual), None
