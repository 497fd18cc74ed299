"""Causal self-attention mixer: MHA or GQA over the paged cache, optional window.

Order of operations as in the reference's block
(src/DotLLM.Models/Architectures/TransformerModel.cs:235-302): Q/K/V projections, position
encoding of Q and K, cache write, attention of the new queries over everything cached, output
projection.  scale = 1/sqrt(head_dim) and query head h reads KV head h // (n_heads/n_kv_heads)
(src/DotLLM.Cpu/Kernels/Attention.cs:47,76,106).  The three projections are stacked into one
matrix when the weights are bound, so one product yields q, k and v side by side.
"""
from __future__ import annotations

import math

import torch

from ..config.spec import PartSpec
from ..errors import ConfigError
from ..kernels import ops
from .base import CacheNeed, Mixer, WeightSpec, make_part, register_mixer

# Branch outputs are handed to the residual add in float32.
BRANCH_DTYPE = torch.float32


class AttentionMixer(Mixer):
    """params: ``n_heads``, ``n_kv_heads``, ``head_dim``, ``window`` (None = all keys),
    ``position`` ({"kind", "params"} of a position encoding), optional ``scale``, optional ``score``
    ({"softcap": c, "slopes": [one per head]}: scores are capped and biased by distance before the
    softmax, which sends the mixer to the generic attention kernel)."""

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.n_heads = int(params["n_heads"])
        self.n_kv_heads = int(params["n_kv_heads"])
        self.head_dim = int(params["head_dim"])
        if self.n_heads % self.n_kv_heads:
            raise ConfigError(f"{self.n_heads} query heads are not a multiple of {self.n_kv_heads} KV heads")
        self.window = params.get("window")
        self.scale = float(params.get("scale", 1.0 / math.sqrt(self.head_dim)))
        pos = params.get("position") or {"kind": "none", "params": {}}
        self.position = make_part("position_encoding", PartSpec(pos["kind"], pos.get("params", {})),
                                  hidden_size, runtime)
        self.graph_safe = bool(getattr(self.position, "graph_safe", True))
        score = params.get("score") or {}
        slopes = score.get("slopes")
        if slopes is not None and len(slopes) != self.n_heads:
            raise ConfigError(f"score slopes: {len(slopes)} values for {self.n_heads} heads")
        self.score_hook = ops.ScoreHook(score.get("softcap", 0.0),
                                        None if slopes is None else torch.tensor(list(slopes), dtype=torch.float32,
                                                                                 device=runtime.device))
        self.q_dim = self.n_heads * self.head_dim
        self.kv_dim = self.n_kv_heads * self.head_dim
        self.w_qkv = None
        self.w_o = None

    def weight_specs(self):
        h = self.hidden_size
        return {"q_proj.weight": WeightSpec((self.q_dim, h)),
                "k_proj.weight": WeightSpec((self.kv_dim, h)),
                "v_proj.weight": WeightSpec((self.kv_dim, h)),
                "o_proj.weight": WeightSpec((h, self.q_dim))}

    def bind(self, tensors):
        self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                                tensors["v_proj.weight"]], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()

    def weight_bytes(self):
        return (self.w_qkv.numel() + self.w_o.numel()) * self.w_qkv.element_size()

    def cache_need(self):
        return CacheNeed("kv", n_kv_heads=self.n_kv_heads, head_dim=self.head_dim, window=self.window)

    takes_scaled_rows = True                    # x goes straight into the Q/K/V product

    def forward(self, x, step, cache_view):
        qd, kvd = self.q_dim, self.kv_dim
        fused = self.position.fused_rotary()
        if cache_view.writes and fused is not None:
            # a prompt step: rotation and cache write in the product's epilogue, then attention over the cache
            q = ops.qkv_rope_cache(x, self.w_qkv, fused[0], fused[1], fused[2], step.token_seq, step.token_pos,
                                   cache_view.block_table, cache_view.k, cache_view.v, self.n_heads, self.n_kv_heads,
                                   self.head_dim)
            if q is not None:
                a = ops.attention(q, cache_view.k, cache_view.v, step.token_seq, step.token_pos, cache_view.block_table,
                                  self.n_heads, self.n_kv_heads, self.head_dim, self.scale, int(self.window or 0),
                                  plan=step.attention_plan, score_hook=self.score_hook if self.score_hook else None)
                return ops.linear(a, self.w_o, out_dtype=BRANCH_DTYPE, resident=True, lazy=True)
        if cache_view.writes:
            qkv = ops.linear(x, self.w_qkv, resident=True)
            q, k, v = qkv[:, :qd], qkv[:, qd:qd + kvd], qkv[:, qd + kvd:]
        else:                                   # reads another execution's cache: only queries
            q, k, v = ops.linear(x, self.w_qkv[:qd], resident=True), None, None
        if fused is None:
            self.position.apply(q, k, step.token_pos)
            cos = sin = None
            rotary_dim = 0
        else:
            cos, sin, rotary_dim = fused
        # rotation, cache write and attention: one kernel for a decode step, two otherwise
        a = ops.rope_cache_attention(q, k, v, cos, sin, rotary_dim, step.token_seq, step.token_pos,
                                     cache_view.block_table, cache_view.k, cache_view.v,
                                     self.n_heads, self.n_kv_heads, self.head_dim, self.scale,
                                     int(self.window or 0), plan=step.attention_plan,
                                     score_hook=self.score_hook if self.score_hook else None)
        return ops.linear(a, self.w_o, out_dtype=BRANCH_DTYPE, resident=True, lazy=True)


register_mixer("attention", AttentionMixer)
