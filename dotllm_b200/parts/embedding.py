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

    def forward(self, step):
        """The step's tokens (``step.tokens`` int32 [T]) -> float32 [T, H]: the start of the residual
        stream.  An embedding gets the whole StepContext: one that also encodes positions reads
        ``step.token_pos``."""
        return ops.gather_rows(self.table, step.tokens)


class LinearHead(Part):
    """params: ``vocab_size``.  Whether its matrix is the embedding table is the model description's
    business (``ModelSpec.shared_weights``): the part is handed a [vocab, hidden] matrix either way."""

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.vocab_size = int(params["vocab_size"])
        self.weight = None

    def weight_specs(self):
        return {"weight": WeightSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors):
        w = tensors["weight"]
        self.weight = w if w.is_contiguous() else w.contiguous()

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    takes_scaled_rows = True                    # x goes straight into the product

    def forward(self, x):
        """[R, H] in the run dtype -> float32 logits [R, vocab]."""
        return ops.linear(x, self.weight, out_dtype=torch.float32, resident=True)


register_embedding("token_embedding", TokenEmbedding)
register_head("linear_head", LinearHead)
