"""Typed configuration of the Llama dense decoder, read from config.json's own keys.

Field by field this is the reference's ``ModelConfig`` + ``RoPEConfig``
(src/DotLLM.Core/Models/ModelConfig.cs:10-68,
src/DotLLM.Core/PositionEncoding/RoPEConfig.cs:17-26) as filled by
``GgufModelConfigExtractor.Extract``
(src/DotLLM.Models/Gguf/GgufModelConfigExtractor.cs:18-68, 100-159), with the
HuggingFace key names.  Defaults for absent keys are the extractor's.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Optional

from ..errors import ConfigError


@dataclass(frozen=True)
class Llama3RopeScaling:
    """``rope_scaling`` with ``rope_type: "llama3"``.  The reference parses scaling
    keys and never applies them (GgufModelConfigExtractor.cs:128-147); the
    rescaling itself is defined in ``parts.rotary``."""
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int
    rope_type: str = "llama3"


def _need(d, key, kind=int):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json lacks required key {key!r}")
    try:
        return kind(d[key])
    except (TypeError, ValueError) as exc:
        raise ConfigError(f"config.json key {key!r} = {d[key]!r} is not {kind.__name__}") from exc


def _token_ids(value):
    if value is None:
        return ()
    if isinstance(value, (list, tuple)):
        return tuple(int(v) for v in value)
    return (int(value),)


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[Llama3RopeScaling]
    tie_word_embeddings: bool
    hidden_act: str = "silu"
    bos_token_id: Optional[int] = None
    eos_token_id: tuple = ()
    architecture: str = "LlamaForCausalLM"

    # ---- derived sizes (TransformerModel.cs:152)
    @property
    def q_dim(self):
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self):
        return self.num_key_value_heads * self.head_dim

    @classmethod
    def from_dict(cls, d):
        heads = _need(d, "num_attention_heads")
        hidden = _need(d, "hidden_size")
        if heads <= 0:
            raise ConfigError("num_attention_heads must be positive")
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"hidden_size {hidden} is not a multiple of num_attention_heads "
                                  f"{heads} and head_dim is not given")
            head_dim = hidden // heads                       # GgufModelConfigExtractor.cs:32-33
        scaling = d.get("rope_scaling")
        if scaling is not None:
            if not isinstance(scaling, dict):
                raise ConfigError("rope_scaling must be an object or null")
            kind = scaling.get("rope_type", scaling.get("type"))
            if kind in (None, "default"):
                scaling = None
            elif kind == "llama3":
                scaling = Llama3RopeScaling(
                    factor=_need(scaling, "factor", float),
                    low_freq_factor=_need(scaling, "low_freq_factor", float),
                    high_freq_factor=_need(scaling, "high_freq_factor", float),
                    original_max_position_embeddings=_need(scaling, "original_max_position_embeddings"))
            else:
                raise ConfigError(f"unsupported rope_scaling type {kind!r} (supported: 'llama3')")
        cfg = cls(
            vocab_size=_need(d, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_need(d, "intermediate_size"),
            num_hidden_layers=_need(d, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=int(d.get("num_key_value_heads") or heads),   # extractor :28
            head_dim=int(head_dim),
            max_position_embeddings=int(d.get("max_position_embeddings") or 2048),   # :34
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-5)),                  # :36
            rope_theta=float(d.get("rope_theta", 10000.0)),                   # :109
            rope_scaling=scaling,
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            hidden_act=str(d.get("hidden_act", "silu")),
            bos_token_id=None if d.get("bos_token_id") is None else int(d["bos_token_id"]),
            eos_token_id=_token_ids(d.get("eos_token_id")),
        )
        if d.get("attention_bias") or d.get("mlp_bias"):
            raise ConfigError("attention_bias / mlp_bias are not supported: the Llama path has no biases")
        cfg.validate()
        return cfg

    def validate(self):
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim",
                    "max_position_embeddings"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{key} must be positive, got {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads:      # Attention.cs:72-74
            raise ConfigError(f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                              f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:                                         # RoPE.cs:47-48
            raise ConfigError(f"head_dim must be even, got {self.head_dim}")
        if not self.rms_norm_eps > 0:
            raise ConfigError("rms_norm_eps must be positive")
        if not self.rope_theta > 0:
            raise ConfigError("rope_theta must be positive")
        if self.hidden_act != "silu":                                 # ModelConfig.cs:49
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported (Llama uses 'silu')")
        s = self.rope_scaling
        if s is not None:
            if s.factor <= 0 or s.high_freq_factor <= s.low_freq_factor or s.low_freq_factor <= 0 \
                    or s.original_max_position_embeddings <= 0:
                raise ConfigError(f"invalid llama3 rope_scaling {s}")

    def to_dict(self):
        """The config.json content that reads back to this configuration."""
        d = asdict(self)
        arch = d.pop("architecture")
        d["architectures"] = [arch]
        d["model_type"] = "llama"
        eos = d.pop("eos_token_id")
        if eos:
            d["eos_token_id"] = list(eos) if len(eos) > 1 else eos[0]
        if d["bos_token_id"] is None:
            d.pop("bos_token_id")
        return d
