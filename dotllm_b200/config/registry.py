"""The one registry from an architecture's name to its configuration type and model builder.

The reference's registry is the ``Architecture`` enum, a string switch in the
metadata extractor and ``IModelArchitecture.CreateModel``
(src/DotLLM.Core/Configuration/Architecture.cs:6-22,
src/DotLLM.Models/Gguf/GgufModelConfigExtractor.cs:70-81,
src/DotLLM.Models/Architectures/TransformerArchitecture.cs:26-43).
Here a name from ``config.json``'s ``architectures`` list maps to a typed
configuration class and a function from that configuration to a ``ModelSpec``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

from ..errors import ConfigError
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_type: type            # has ``from_dict(dict)`` and ``to_dict()``
    build_spec: Callable         # config -> ModelSpec
    model_types: tuple = ()      # accepted ``model_type`` values when ``architectures`` is absent


_ARCHITECTURES: dict = {}


def register_architecture(name, config_type, build_spec, model_types=()):
    """Add an architecture.  Registering a name twice replaces the earlier entry."""
    _ARCHITECTURES[name] = Architecture(name, config_type, build_spec, tuple(model_types))
    return _ARCHITECTURES[name]


def registered_architectures():
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def _ensure_builtin():
    # Built-in architectures register themselves on import.
    from ..models import llama  # noqa: F401


def resolve_architecture(config_dict) -> Architecture:
    _ensure_builtin()
    names = config_dict.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    for name in names:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    model_type = config_dict.get("model_type")
    if not names and model_type is not None:
        for arch in _ARCHITECTURES.values():
            if model_type in arch.model_types:
                return arch
    asked = names if names else ([model_type] if model_type else [])
    raise ConfigError(f"unknown architecture {asked!r}; registered: {registered_architectures()}")


def config_from_dict(config_dict):
    """The typed configuration of whichever architecture ``config_dict`` names."""
    if not isinstance(config_dict, dict):
        raise ConfigError("config.json must hold a JSON object")
    arch = resolve_architecture(config_dict)
    return arch.config_type.from_dict(config_dict)


def load_config(folder):
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"no config.json in {folder}")
    try:
        data = json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: not valid JSON ({exc})") from exc
    return config_from_dict(merge_generation_config(data, Path(folder) / "generation_config.json"))


def merge_generation_config(data, path):
    """``generation_config.json``, where a folder has one, names the tokens that end generation
    (Llama 3 checkpoints list several there and one in config.json): its ``eos_token_id`` entries come
    first, config.json's follow, duplicates dropped; its ``bos_token_id`` fills a missing one.  The
    reference takes both ids from the tokenizer (src/DotLLM.Tokenizers/ITokenizer.cs:38-41)."""
    if not path.is_file():
        return data
    try:
        gen = json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: not valid JSON ({exc})") from exc
    if not isinstance(gen, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    as_list = lambda v: [] if v is None else (list(v) if isinstance(v, (list, tuple)) else [v])
    merged = []
    for token in as_list(gen.get("eos_token_id")) + as_list(data.get("eos_token_id")):
        if token not in merged:
            merged.append(token)
    out = dict(data)
    if merged:
        out["eos_token_id"] = merged
    if out.get("bos_token_id") is None and gen.get("bos_token_id") is not None:
        out["bos_token_id"] = gen["bos_token_id"]
    return out


def build_spec(config) -> ModelSpec:
    """The model description of a typed configuration, through its architecture's builder."""
    _ensure_builtin()
    for arch in _ARCHITECTURES.values():
        if isinstance(config, arch.config_type) and getattr(config, "architecture", arch.name) == arch.name:
            spec = arch.build_spec(config)
            spec.validate()
            return spec
    raise ConfigError(f"no registered architecture builds a {type(config).__name__}")
