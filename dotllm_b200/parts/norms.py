"""RMSNorm over the float32 residual stream.

y = x / sqrt(mean(x^2) + eps) * gain, eps inside the root, no mean subtraction, gain used as
is (src/DotLLM.Cpu/Kernels/RmsNorm.cs:22-51).  The fused form adds a pending branch output
to the stream first, as the reference's fused_add_rmsnorm does
(native/kernels/fused_add_rmsnorm.cu:9-72).
"""
from __future__ import annotations

from ..kernels import ops
from .base import Norm, WeightSpec, register_norm


class RmsNorm(Norm):
    """params: ``eps``; optional ``gain_init`` for the random-weights mode."""

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.eps = float(params["eps"])
        self.gain = None

    def weight_specs(self):
        return {"weight": WeightSpec((self.hidden_size,), "precise",
                                     tuple(self.params.get("gain_init", ("ones",))))}

    def bind(self, tensors):
        self.gain = tensors["weight"]

    def weight_bytes(self):
        return self.gain.numel() * self.gain.element_size()

    fuses_products = True

    def forward(self, x):
        return ops.add_rmsnorm(x, None, self.gain, self.eps, self.runtime.dtype)

    def add_forward(self, residual, delta, lazy=False):
        return ops.add_rmsnorm(residual, delta, self.gain, self.eps, self.runtime.dtype, lazy=lazy)


register_norm("rmsnorm", RmsNorm)
