"""Dense gated feed-forward (SwiGLU): down(silu(gate(x)) * up(x)).

src/DotLLM.Models/Architectures/TransformerModel.cs:342-382 with the activation of
src/DotLLM.Cpu/Kernels/FusedOps.cs:33-78.  Gate and up are stacked into one matrix when the
weights are bound, so one product feeds the gating kernel.
"""
from __future__ import annotations

import torch

from ..errors import ConfigError
from ..kernels import ops
from .attention import BRANCH_DTYPE
from .base import FeedForward, WeightSpec, register_feed_forward


class GatedFeedForward(FeedForward):
    """params: ``intermediate_size``, ``activation`` ("silu")."""

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.intermediate_size = int(params["intermediate_size"])
        if params.get("activation", "silu") != "silu":
            raise ConfigError(f"gated feed-forward: unsupported activation {params['activation']!r}")
        self.w_gate_up = None
        self.w_down = None

    def weight_specs(self):
        i, h = self.intermediate_size, self.hidden_size
        return {"gate_proj.weight": WeightSpec((i, h)),
                "up_proj.weight": WeightSpec((i, h)),
                "down_proj.weight": WeightSpec((h, i))}

    def bind(self, tensors):
        self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def weight_bytes(self):
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    takes_scaled_rows = True                    # x goes straight into the gate/up product

    def forward(self, x):
        return ops.linear(ops.gated_linear(x, self.w_gate_up, resident=True), self.w_down, out_dtype=BRANCH_DTYPE,
                          resident=True, lazy=True)


register_feed_forward("gated_mlp", GatedFeedForward)
