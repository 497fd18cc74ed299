"""Block arrangements: how a layer's parts meet the residual stream.

"pre_norm" is the reference's wiring, r=h; h=r+mixer(norm(h)); r=h; h=r+ffn(norm(h))
(src/DotLLM.Models/Architectures/TransformerModel.cs:185-392).  As in the reference's GPU path
(src/DotLLM.Cuda/CudaTransformerModel.cs:252-286) each residual add is folded into the norm
that follows it, across the layer boundary too: a block returns its last branch output still
to be added ("pending"), and whoever normalises next adds it.
"""
from __future__ import annotations

from .base import Arrangement, normalised_for, register_arrangement


class PreNormBlock(Arrangement):
    needs = ("mixer_norm", "mixer", "feed_forward_norm", "feed_forward")
    narrows = True

    def forward(self, residual, pending, step, cache_view, keep_rows=None):
        n = normalised_for(self.mixer, self.mixer_norm, residual, pending)
        a = self.mixer.forward(n, step, cache_view)          # every token: the cache needs all keys and values
        if keep_rows is not None:
            # nothing after this layer reads the other rows: the output projection, the second norm and
            # the feed-forward run on the kept rows only
            from ..kernels import ops
            residual = ops.gather_rows(residual, keep_rows)
            a = ops.narrow_rows(a, keep_rows)
        n = normalised_for(self.feed_forward, self.feed_forward_norm, residual, a)
        return residual, self.feed_forward.forward(n)


register_arrangement("pre_norm", PreNormBlock)
