"""Rotary position encoding: frequency table, optional llama3 rescaling, half-split rotation.

Frequencies f_i = theta^(-2i/d), angle = pos * f_i, cos/sin tabulated per position
(src/DotLLM.Cpu/Kernels/RoPE.cs:44-86).  Tensors in HuggingFace order pair (x[i], x[i+d/2])
(RoPE.cs:211-257; src/DotLLM.Core/Configuration/RoPEType.cs:11-23).  The reference parses
scaling keys and applies none (src/DotLLM.Cpu/Kernels/RoPE.md:303); the "llama3" rule here is
the one published with the Llama 3.1 checkpoints: wavelengths below P/high keep their
frequency, above P/low are divided by ``factor``, and those between are blended linearly in
P/wavelength.  Tables are computed once in float64 and rounded to float32.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from ..errors import ConfigError
from ..kernels import ops
from .base import PositionEncoding, register_position_encoding


def rotary_frequencies(rotary_dim, theta, scaling=None):
    """float64 [rotary_dim/2].  ``scaling``: None or a dict with ``rope_type`` "llama3"."""
    i = np.arange(rotary_dim // 2, dtype=np.float64)
    freq = np.power(float(theta), -2.0 * i / rotary_dim)
    if not scaling:
        return freq
    kind = scaling.get("rope_type")
    if kind != "llama3":
        raise ConfigError(f"unsupported rotary scaling {kind!r}")
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    wavelen = 2.0 * math.pi / freq
    smooth = (orig / wavelen - low) / (high - low)
    blended = (1.0 - smooth) * freq / factor + smooth * freq
    return np.where(wavelen < orig / high, freq, np.where(wavelen > orig / low, freq / factor, blended))


_TABLES: dict = {}


class RotaryEncoding(PositionEncoding):
    """params: ``rotary_dim``, ``theta``, ``max_positions``, ``scaling`` (None or dict)."""

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.rotary_dim = int(params["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ConfigError(f"rotary_dim must be positive and even, got {self.rotary_dim}")
        self.max_positions = int(params["max_positions"])
        scaling = params.get("scaling")
        key = (self.rotary_dim, float(params["theta"]), self.max_positions,
               tuple(sorted(scaling.items())) if scaling else None, str(runtime.device))
        if key not in _TABLES:                      # layers with equal parameters share one table
            freq = rotary_frequencies(self.rotary_dim, params["theta"], scaling)
            angle = np.arange(self.max_positions, dtype=np.float64)[:, None] * freq[None, :]
            _TABLES[key] = tuple(torch.from_numpy(f(angle).astype(np.float32)).to(runtime.device).contiguous()
                                 for f in (np.cos, np.sin))
        self.cos, self.sin = _TABLES[key]

    def fused_rotary(self):
        return self.cos, self.sin, self.rotary_dim

    def apply(self, q, k, positions):
        """Unfused form: rotate q and k in place (each [T, heads*head_dim])."""
        hd = int(self.params.get("head_dim", self.rotary_dim))
        for x in (q, k):
            if x is None:
                continue
            ops.rope_cache_write(x, None, None, self.cos, self.sin, self.rotary_dim, None, positions,
                                 None, None, None, x.shape[1] // hd, 1, hd, write_cache=False)


class NoPositionEncoding(PositionEncoding):
    """Queries and keys carry no position information."""

    def apply(self, q, k, positions):
        return None


register_position_encoding("rotary", RotaryEncoding)
register_position_encoding("none", NoPositionEncoding)
