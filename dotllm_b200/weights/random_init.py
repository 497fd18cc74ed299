"""Random-weights mode: fill a model from a configuration and a seed, or write it as a folder.

The reference has no such mode (all its model tests use downloaded checkpoints,
tests/DotLLM.Tests.Integration/Fixtures/SmallModelFixture.cs:11-20).  Every tensor draws from a
generator seeded by (seed, tensor name), so a tensor's values do not depend on which other
tensors exist or on the order they are made in.  Matrices are N(0, std); norm gains are what
their part declares (ones, or 1 + U(-a, a)).
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from .safetensors_io import save_safetensors


def _name_seed(seed, name):
    h = 0xcbf29ce484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
    return (h ^ (int(seed) * 0x9E3779B97F4A7C15)) & 0x7FFFFFFFFFFFFFFF


def random_tensor(name, spec, seed, device="cpu"):
    """float32 (int32 for index tables) tensor for ``spec``, reproducible from (seed, name)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(_name_seed(seed, name))
    kind = spec.init[0]
    shape = tuple(spec.shape)
    if kind == "normal":
        return torch.randn(shape, generator=gen, dtype=torch.float32, device=device) * float(spec.init[1])
    if kind == "ones":
        return torch.ones(shape, dtype=torch.float32, device=device)
    if kind == "zeros":
        return torch.zeros(shape, dtype=torch.float32, device=device)
    if kind == "one_plus_uniform":
        a = float(spec.init[1])
        return 1.0 + (torch.rand(shape, generator=gen, dtype=torch.float32, device=device) * 2.0 - 1.0) * a
    raise ValueError(f"unknown init {spec.init!r} for tensor {name!r}")


def init_random(model, seed, on_device=False):
    """Bind ``model`` to random tensors without touching the disk.  With ``on_device`` the
    numbers are drawn by the device's generator (fast for multi-GB models; a different stream
    than the CPU's)."""
    expected, _ = model.expected_weights()
    device = model.runtime.device if on_device else "cpu"
    model.bind(lambda name: random_tensor(name, expected[name], seed, device))
    return model


def write_random_model(folder, config, seed, dtype=torch.bfloat16, spec_builder=None):
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a typed configuration).

    Matrices are stored in ``dtype`` (bfloat16 or float32); norm gains and other "precise"
    tensors are stored in float32."""
    from ..config.registry import build_spec
    from ..models.decoder import DecoderModel
    from ..parts.base import Runtime
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    spec = spec_builder(config) if spec_builder else build_spec(config)
    skeleton = DecoderModel(spec, Runtime(dtype, torch.device("meta")))
    expected, _ = skeleton.expected_weights()
    tensors = {}
    for name, wspec in expected.items():
        t = random_tensor(name, wspec, seed)
        tensors[name] = t.to(dtype) if wspec.role == "matrix" else t
    save_safetensors(folder / "model.safetensors", tensors, metadata={"format": "pt", "seed": seed})
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=2))
    return folder
