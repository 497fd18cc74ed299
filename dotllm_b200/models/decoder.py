"""The generic decoder: runs any model description over a step of tokens.

Embedding, then the scheduled layer executions, then the final norm and the head on the rows
whose logits are wanted - the reference's forward pass
(src/DotLLM.Models/Architectures/TransformerModel.cs:134-425), with its GPU variant's habit of
computing the head only where logits are needed (src/DotLLM.Cuda/CudaTransformerModel.cs:289-297).
Nothing in this file knows an architecture's name.
"""
from __future__ import annotations

import torch

from ..cache.model_cache import ModelCache
from ..config.spec import ModelSpec
from ..kernels import ops
from ..parts.base import Runtime, make_arrangement, make_part, normalised_for


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        spec.validate()
        self.spec = spec
        self.runtime = runtime
        h = spec.hidden_size
        self.embedding = make_part("embedding", spec.embedding, h, runtime)
        self.blocks = []
        self._named_parts = [(spec.embedding.prefix, self.embedding)]
        for layer in spec.layers:
            built = {p.name: make_part(p.family, p.spec, h, runtime) for p in layer.parts}
            self.blocks.append(make_arrangement(layer.arrangement, built))
            self._named_parts += [(p.spec.prefix, built[p.name]) for p in layer.parts]
        self.final_norm = make_part("norm", spec.final_norm, h, runtime)
        self.head = make_part("head", spec.head, h, runtime)
        self._named_parts += [(spec.final_norm.prefix, self.final_norm), (spec.head.prefix, self.head)]
        # may a step be captured as a CUDA graph?  Only if every part just launches work (Part.graph_safe)
        self.graph_safe = all(getattr(part, "graph_safe", True) for _, part in self._named_parts) and \
            all(getattr(block, "graph_safe", True) for block in self.blocks)
        self.bound = False

    # ------------------------------------------------------------- weights
    def named_parts(self):
        """(prefix, part) for every part that may own tensors."""
        return list(self._named_parts)

    def expected_weights(self):
        """Full tensor name -> WeightSpec, and the set of names that may be present and are ignored."""
        expected, optional = {}, set()
        for prefix, part in self._named_parts:
            for local, spec in part.weight_specs().items():
                expected[prefix + local] = spec
            optional |= {prefix + local for local in part.optional_names()}
        for name, source in self.spec.shared_weights:
            if name not in expected or source not in expected:
                raise ValueError(f"shared weight {name!r} = {source!r}: both must be tensors that parts declare")
            if tuple(expected[name].shape) != tuple(expected[source].shape) or expected[name].role != expected[source].role:
                raise ValueError(f"shared weight {name!r} and {source!r} differ in shape or role")
            del expected[name]                              # not looked for in a checkpoint ...
            optional.add(name)                              # ... and a copy stored there is tolerated
        return expected, optional

    def convert(self, spec, tensor):
        """A loaded tensor in the dtype its role asks for, on the device."""
        t = tensor.to(self.runtime.device)
        if spec.role == "matrix":
            return t.to(self.runtime.dtype)
        if spec.role == "precise":
            return t.to(torch.float32)
        if spec.role == "index":
            return t.to(torch.int32)
        raise ValueError(f"unknown weight role {spec.role!r}")

    def bind(self, fetch):
        """Give every part its tensors.  ``fetch(full_name)`` returns the stored tensor."""
        shared = dict(self.spec.shared_weights)
        converted = {}                                      # full name -> tensor, so that a shared tensor is one object

        def get(name, spec):
            name = shared.get(name, name)
            if name not in converted:
                converted[name] = self.convert(spec, fetch(name))
            return converted[name]

        for prefix, part in self._named_parts:
            part.bind({local: get(prefix + local, spec) for local, spec in part.weight_specs().items()})
        self.bound = True

    def weight_bytes_per_step(self):
        """Bytes of weights a decode step reads: every matrix once; the embedding table only
        when the head shares it (a lookup touches a few rows)."""
        return sum(part.weight_bytes() for _, part in self._named_parts)

    # --------------------------------------------------------------- cache
    def cache_needs(self):
        return [self.blocks[e.layer].cache_need() for e in self.spec.schedule]

    def new_cache(self, max_tokens, max_sequences=None):
        return ModelCache(self.cache_needs(), [e.cache_of for e in self.spec.schedule], self.runtime,
                          max_tokens, max_sequences)

    # ------------------------------------------------------------- forward
    def forward(self, step, cache):
        """Logits float32 [wanted rows, vocab] of one step (see engine.step)."""
        residual = self.embedding.forward(step)
        pending = None
        # Logits are wanted at some rows only (a prompt's last token): the last layer in the order of
        # running still caches every token, but may hand on the wanted rows alone.
        some = 0 < step.n_wanted and not step.want_all
        narrowed = False
        last = len(self.spec.schedule) - 1
        for e, entry in enumerate(self.spec.schedule):
            view = cache.view(e, step.block_tables, step.slots)
            block = self.blocks[entry.layer]
            if e == last and some and block.narrows:
                residual, pending = block.forward(residual, pending, step, view, keep_rows=step.want_rows)
                narrowed = True
            else:
                residual, pending = block.forward(residual, pending, step, view)
        if step.n_wanted == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.runtime.device)
        if some and not narrowed:
            if isinstance(pending, ops.PendingProduct) and pending.add_into(residual):
                pending = None                    # the last product added itself into the stream
            residual = ops.gather_rows(residual, step.want_rows)
            pending = ops.narrow_rows(pending, step.want_rows)
        return self.head.forward(normalised_for(self.head, self.final_norm, residual, pending))
