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
class LayerSpec:
    """One layer that owns weights: an arrangement of a mixer, a feed-forward and their norms."""
    arrangement: str            # registered block arrangement, e.g. "pre_norm"
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec


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

    def validate(self) -> None:
        from ..errors import ConfigError
        if not self.schedule:
            raise ConfigError("the schedule names no layer")
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
