"""Interfaces of the parts a layer is made of, and the registries that build them by kind.

A part knows its own sizes and constants (given as ``params``) and nothing about the model
it sits in.  The reference declares the same seams as ``IAttentionStrategy``
(src/DotLLM.Core/Attention/IAttentionStrategy.cs:9-27) and ``IPositionEncoding``
(src/DotLLM.Core/PositionEncoding/IPositionEncoding.cs:10-34) but wires its forward pass
around them (docs/ATTENTION.md:5); here the block really runs through the interfaces.

Kinds are registered by name:

    register_mixer("attention", AttentionMixer)
    register_feed_forward("gated_mlp", GatedFeedForward)
    register_norm("rmsnorm", RmsNorm)
    register_position_encoding("rotary", RotaryEncoding)
    register_arrangement("pre_norm", PreNormBlock)

and a ``PartSpec(kind, params, prefix)`` picks one per layer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..errors import ConfigError


@dataclass(frozen=True)
class Runtime:
    """Where and in which precision a model runs."""
    dtype: torch.dtype            # torch.float32 or torch.bfloat16: matrices, activations, cache
    device: torch.device


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part needs.

    role "matrix": operand of a matrix product or a lookup table; converted to the run dtype.
    role "precise": used in 32-bit arithmetic (norm gains); widened to / kept in float32.
    role "index": integer table; kept as int32.
    ``init`` says how the random-weights mode fills it: ("normal", std), ("ones",),
    ("one_plus_uniform", a) or ("zeros",).
    """
    shape: tuple
    role: str = "matrix"
    init: tuple = ("normal", 0.02)


@dataclass(frozen=True)
class CacheNeed:
    """What one execution of a mixer keeps per sequence.

    kind "kv": keys and values per token, ``n_kv_heads`` x ``head_dim`` each; ``window`` None
    keeps every token, an integer keeps the last ``window``.  ``k_dim`` / ``v_dim`` give keys and
    values widths of their own (a compressed or latent cache) and ``dtype`` a storage type of its own
    (default: the run's); the built-in attention kernels take equal widths in the run's type, a mixer
    with other needs reads and writes its pages itself.
    kind "state": a fixed-size tensor of ``state_shape`` / ``state_dtype`` per sequence, zero
    when the sequence starts.
    """
    kind: str
    n_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: tuple = ()
    state_dtype: torch.dtype = torch.float32
    k_dim: Optional[int] = None
    v_dim: Optional[int] = None
    dtype: Optional[torch.dtype] = None

    def key_width(self):
        return self.k_dim or self.head_dim

    def value_width(self):
        return self.v_dim or self.head_dim

    def group_key(self, run_dtype):
        if self.kind == "kv":
            return ("kv", self.n_kv_heads, self.key_width(), self.value_width(), self.window, self.dtype or run_dtype)
        return ("state", tuple(self.state_shape), self.state_dtype)


class Part:
    """Base of every part: declares tensors, receives them, runs.

    ``graph_safe``: the part's forward only launches work on the current stream, so a step may be
    captured as a CUDA graph and replayed.  A part that waits for the device or reads device values
    on the host in its forward (``.tolist()``, ``.item()``, a Python loop over a tensor's values) sets
    it to False; a model that holds such a part runs every step eagerly."""

    graph_safe = True

    def __init__(self, params: dict, hidden_size: int, runtime: Runtime):
        self.params = dict(params)
        self.hidden_size = hidden_size
        self.runtime = runtime

    def weight_specs(self) -> dict:
        """local tensor name -> WeightSpec"""
        return {}

    def optional_names(self) -> set:
        """Local names that a checkpoint may hold and this part ignores."""
        return set()

    def bind(self, tensors: dict) -> None:
        """Receive the declared tensors, already on the device in the dtype their role asks for."""

    def weight_bytes(self) -> int:
        """Bytes of weights that one step reads (for the roofline account)."""
        return 0


class Norm(Part):
    """``fuses_products``: ``add_forward`` also takes ``lazy=True`` and a delta that is a product not yet
    launched (``ops.PendingProduct``), and may then return ``ops.ScaledRows`` instead of a tensor."""
    fuses_products = False

    def forward(self, x):
        """Normalised copy of the float32 stream ``x`` in the run dtype."""
        raise NotImplementedError

    def add_forward(self, residual, delta):
        """residual += delta in place (float32), then the normalised result in the run dtype."""
        raise NotImplementedError


def normalised_for(consumer, norm, residual, pending):
    """The stream, with the branch output ``pending`` (or None) added, normalised by ``norm`` for the
    part ``consumer``.  A part may return its last product unlaunched (``ops.linear(..., lazy=True)``);
    a norm that ``fuses_products`` then lets that product do the addition, and a consumer that
    ``takes_scaled_rows`` (it hands its input straight to ``ops.linear`` / ``ops.gated_linear``) lets its
    first product do the normalisation.  Everyone else gets and gives plain tensors."""
    if pending is None:
        return norm.forward(residual)
    if norm.fuses_products:
        return norm.add_forward(residual, pending, lazy=bool(getattr(consumer, "takes_scaled_rows", False)))
    from ..kernels import ops
    return norm.add_forward(residual, ops.resolve(pending))


class PositionEncoding(Part):
    """Position information for a mixer's queries and keys.

    ``fused_rotary()`` returns (cos, sin, rotary_dim) when the encoding is a rotation that the
    cache-write kernel can apply on the fly, else None, in which case the mixer calls
    ``apply(q, k, positions)`` before the plain cache write."""

    def fused_rotary(self):
        return None

    def apply(self, q, k, positions):
        """Encode in place.  q [T, nh*hd], k [T, nkv*hd] (k may be None), positions int32 [T]."""
        raise NotImplementedError


class Mixer(Part):
    """Mixes information across the tokens of a sequence (attention, recurrence, ...)."""

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def forward(self, x, step, cache_view):
        """x [T, H] in the run dtype -> the branch output [T, H] (run dtype or float32; it may be a
        last product not yet launched, ``ops.linear(..., lazy=True)``).  A mixer that sets
        ``takes_scaled_rows`` hands x straight to ``ops.linear`` / ``ops.gated_linear`` and may be given
        ``ops.ScaledRows`` instead of a tensor.

        ``step`` is the engine's StepContext (token -> sequence map, positions, lengths);
        ``cache_view`` gives this execution's storage (``LayerCacheView``) or None."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x):
        """x [T, H] in the run dtype -> the branch output [T, H]; ``takes_scaled_rows`` and unlaunched
        last products as for a mixer."""
        raise NotImplementedError


class Arrangement:
    """How a layer's parts and the residual stream are wired.  ``parts`` maps the names of the
    layer's description to the built parts; ``needs`` lists the names this arrangement cannot do
    without.  ``cached_mixer`` names the part whose ``cache_need()`` the layer's cache is made for
    (None: the layer keeps nothing).  ``narrows``: ``forward`` also takes ``keep_rows`` (int32 row
    indices on the device): when the model gives them (the last layer of a step whose logits are
    wanted at some rows only), the arrangement returns the stream and the pending branch for those rows
    alone, in their order, and may skip whatever only the other rows would need - but it must still put
    every token's keys, values and state into the cache."""
    needs = ()
    cached_mixer = "mixer"
    narrows = False
    graph_safe = True            # as Part.graph_safe: the arrangement's own forward waits for nothing

    def __init__(self, parts: dict):
        lacking = [n for n in self.needs if n not in parts]
        if lacking:
            raise ConfigError(f"arrangement {type(self).__name__} needs parts {list(self.needs)}; the layer lacks {lacking}")
        self.parts = dict(parts)
        for name, part in parts.items():                    # the usual names as attributes
            setattr(self, name, part)

    def cache_need(self):
        mixer = self.parts.get(self.cached_mixer) if self.cached_mixer else None
        return mixer.cache_need() if mixer is not None else None

    def forward(self, residual, pending, step, cache_view):
        """Returns (residual, pending): the float32 stream and a branch output not yet added.
        (An arrangement that ``narrows`` also accepts ``keep_rows=None``.)"""
        raise NotImplementedError


_REGISTRIES = {"mixer": {}, "feed_forward": {}, "norm": {}, "position_encoding": {}, "arrangement": {},
               "embedding": {}, "head": {}}


def _register(family, kind, cls):
    _REGISTRIES[family][kind] = cls
    return cls


def register_mixer(kind, cls):
    return _register("mixer", kind, cls)


def register_feed_forward(kind, cls):
    return _register("feed_forward", kind, cls)


def register_norm(kind, cls):
    return _register("norm", kind, cls)


def register_position_encoding(kind, cls):
    return _register("position_encoding", kind, cls)


def register_arrangement(kind, cls):
    return _register("arrangement", kind, cls)


def register_embedding(kind, cls):
    return _register("embedding", kind, cls)


def register_head(kind, cls):
    return _register("head", kind, cls)


def registered(family):
    _ensure_builtin()
    return sorted(_REGISTRIES[family])


def _ensure_builtin():
    from . import norms, rotary, attention, feed_forward, blocks, embedding  # noqa: F401


def make_part(family, spec, hidden_size, runtime):
    """Build the part a PartSpec names."""
    _ensure_builtin()
    try:
        cls = _REGISTRIES[family][spec.kind]
    except KeyError:
        raise ConfigError(f"no {family} of kind {spec.kind!r}; registered: "
                          f"{sorted(_REGISTRIES[family])}") from None
    return cls(spec.params, hidden_size, runtime)


def make_arrangement(kind, parts):
    """``parts``: name -> built part, in the layer description's order."""
    _ensure_builtin()
    try:
        cls = _REGISTRIES["arrangement"][kind]
    except KeyError:
        raise ConfigError(f"no block arrangement {kind!r}; registered: "
                          f"{sorted(_REGISTRIES['arrangement'])}") from None
    return cls(parts)
