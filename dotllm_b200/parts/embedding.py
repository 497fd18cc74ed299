"""Token embedding and the output head.

Embedding: h[t] = E[token[t]], no scale
(src/DotLLM.Models/Architectures/TransformerModel.cs:729-749).  Head: logits = n W^T in
float32 without bias or soft-cap (TransformerModel.cs:411-416); a tied head uses the embedding
table (src/DotLLM.Models/Architectures/TransformerWeights.cs:205-220).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part, WeightSpec, register_embedding, register_head


class TokenEmbedding(Part):
    """params: ``vocab_size``."""

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.vocab_size = int(params["vocab_size"])
        self.table = None

    def weight_specs(self):
        return {"weight": WeightSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors):
        self.table = tensors["weight"].contiguous()

    def forward(self, token_ids):
        """int32 [T] -> float32 [T, H]: the start of the residual stream."""
        return ops.gather_rows(self.table, token_ids)


class LinearHead(Part):
    """params: ``vocab_size``, ``tied`` (use the embedding table)."""

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.vocab_size = int(params["vocab_size"])
        self.tied = bool(params.get("tied", False))
        self.weight = None

    def weight_specs(self):
        return {} if self.tied else {"weight": WeightSpec((self.vocab_size, self.hidden_size))}

    def optional_names(self):
        return {"weight"} if self.tied else set()

    def bind(self, tensors):
        if not self.tied:
            self.weight = tensors["weight"].contiguous()

    def tie(self, table):
        self.weight = table

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    takes_scaled_rows = True                    # x goes straight into the product

    def forward(self, x):
        """[R, H] in the run dtype -> float32 logits [R, vocab]."""
        return ops.linear(x, self.weight, out_dtype=torch.float32, resident=True)


register_embedding("token_embedding", TokenEmbedding)
register_head("linear_head", LinearHead)
