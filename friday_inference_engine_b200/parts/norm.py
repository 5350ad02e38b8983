"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * weight, the mean taken in fp32.

Reference: rmsNormKernel (cuda_math_kernels.cu:280-321), friday_cpu::rmsNorm
(cpu_ops.cpp:10-24).
"""
from .. import ops
from .base import Part, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    category = "norm"

    def __init__(self, env, eps, width=None):
        super().__init__(env)
        self.eps = float(eps)
        self.width = int(width or env.width)
        self.declare("weight", (self.width,), init="one")

    def forward(self, x):
        return ops.rmsnorm(x, self.tensors["weight"], self.eps)

    def as_rmsnorm(self):
        return self.tensors["weight"], self.eps
