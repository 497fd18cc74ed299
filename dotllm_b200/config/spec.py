"""Architecture-independent description of a model: parts, layers and the order they run in.

An architecture's builder turns its typed configuration into a ``ModelSpec``.
Everything below the builder (weights, cache, engine, replay) reads only the
spec, never the architecture's name.  The reference reaches the same end with
one parameterised ``TransformerModel`` whose optional branches are keyed on the
configuration (src/DotLLM.Models/Architectures/TransformerModel.cs:134-425);
here each branch is a part chosen per layer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered kind, its sizes and constants, and where its tensors live.

    ``prefix`` is prepended to the part's local tensor names
    (``"model.layers.3.self_attn."`` + ``"q_proj.weight"``).
    """
    kind: str
    params: dict = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerPart:
    """One part of a layer: the name its arrangement knows it by, its family ("mixer",
    "feed_forward" or "norm") and its description."""
    name: str
    family: str
    spec: PartSpec


@dataclass(frozen=True)
class LayerSpec:
    """One layer that owns weights: an arrangement and the named parts it wires together, in the order
    their tensors are declared.  An arrangement asks for the names it needs: "pre_norm" wants
    ``mixer_norm``, ``mixer``, ``feed_forward_norm`` and ``feed_forward``; a layer without a
    feed-forward, or one with four norms, is another arrangement over another list."""
    arrangement: str            # registered block arrangement, e.g. "pre_norm"
    parts: tuple                # of LayerPart

    def part(self, name):
        for p in self.parts:
            if p.name == name:
                return p.spec
        raise KeyError(name)


def pre_norm_layer(mixer, feed_forward, mixer_norm, feed_forward_norm, arrangement="pre_norm"):
    """The usual layer: norm -> mixer -> norm -> feed-forward, each branch added to the stream."""
    return LayerSpec(arrangement, (LayerPart("mixer_norm", "norm", mixer_norm), LayerPart("mixer", "mixer", mixer),
                                   LayerPart("feed_forward_norm", "norm", feed_forward_norm),
                                   LayerPart("feed_forward", "feed_forward", feed_forward)))


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.

    ``layer`` indexes ``ModelSpec.layers`` and may occur in several entries
    (shared weights).  ``cache_of`` is ``None`` when the execution keeps a cache
    of its own, or the index of an earlier schedule entry whose cache it reads
    without writing.
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple
    schedule: tuple
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: tuple = ()
    bos_token_id: Optional[int] = None
    # (tensor a part declares, tensor it is the same as): the first is not looked for in a
    # checkpoint, its part is handed the second's tensor (a head tied to the embedding table)
    shared_weights: tuple = ()

    def validate(self) -> None:
        from ..errors import ConfigError
        if not self.schedule:
            raise ConfigError("the schedule names no layer")
        for layer in self.layers:
            names = [p.name for p in layer.parts]
            if len(set(names)) != len(names):
                raise ConfigError(f"a layer names a part twice: {names}")
            for p in layer.parts:
                if p.family not in ("mixer", "feed_forward", "norm"):
                    raise ConfigError(f"layer part {p.name!r} has unknown family {p.family!r}")
        for n, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ConfigError(f"schedule entry {n} names layer {entry.layer}, "
                                  f"but there are {len(self.layers)} layers")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < n:
                    raise ConfigError(f"schedule entry {n} reads the cache of entry "
                                      f"{entry.cache_of}, which does not run before it")
                if self.schedule[entry.cache_of].cache_of is not None:
                    raise ConfigError(f"schedule entry {n} reads the cache of entry "
                                      f"{entry.cache_of}, which keeps none of its own")


def as_plain(value: Any) -> Any:
    """Dataclasses and tuples to JSON-ready dicts and lists (for logs and bench records)."""
    from dataclasses import asdict, is_dataclass
    if is_dataclass(value):
        return {k: as_plain(v) for k, v in asdict(value).items()}
    if isinstance(value, (list, tuple)):
        return [as_plain(v) for v in value]
    if isinstance(value, dict):
        return {k: as_plain(v) for k, v in value.items()}
    return value
