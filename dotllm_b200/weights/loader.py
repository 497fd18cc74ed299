"""Resolve a model's tensors by name from safetensors files and check them against the model.

The reference indexes the GGUF tensor dictionary by name, so a missing tensor surfaces as a
KeyNotFoundException on first use (src/DotLLM.Models/Architectures/TransformerWeights.cs:183-205).
Here everything is compared up front and ONE error lists all missing tensors, all unexpected
tensors and all wrong shapes.  Tensors come back in their stored precision: bfloat16 stays
bfloat16, 32-bit stays 32-bit, integer tables become int32; conversion to a part's compute dtype
is the model's business (``DecoderModel.convert``).
"""
from __future__ import annotations

import torch

from ..errors import WeightsError
from .safetensors_io import open_model_files

_FLOAT_TAGS = {"F32", "BF16", "F16", "F64"}
_INT_TAGS = {"I64", "I32", "I16", "I8", "U8"}


def stored_tensor(file, name):
    """The tensor as the loader keeps it: bfloat16 and float32 as stored; float16 widened to
    float32 (exact); float64 narrowed to float32; integers to int32."""
    tag = file.dtype_tag(name)
    t = file.tensor(name)
    if tag in ("F32", "BF16"):
        return t
    if tag in ("F16", "F64"):
        return t.to(torch.float32)
    if tag in _INT_TAGS:
        return t.to(torch.int32)
    raise WeightsError(f"tensor {name!r}: dtype {tag} cannot be a model weight")


def check_names_and_shapes(available, expected, optional=()):
    """``available``: name -> shape found; ``expected``: name -> WeightSpec.  Raises one
    WeightsError naming every problem."""
    missing = sorted(n for n in expected if n not in available)
    unexpected = sorted(n for n in available if n not in expected and n not in optional)
    wrong = sorted((n, tuple(expected[n].shape), tuple(available[n]))
                   for n in expected if n in available and tuple(available[n]) != tuple(expected[n].shape))
    if not (missing or unexpected or wrong):
        return
    lines = ["the checkpoint does not match the model:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}): " +
                     ", ".join(f"{n} expected {list(e)} found {list(f)}" for n, e, f in wrong))
    err = WeightsError("\n".join(lines))
    err.missing, err.unexpected, err.wrong_shapes = missing, unexpected, wrong
    raise err


def load_into(model, folder):
    """Bind ``model``'s parts to the tensors of the model folder."""
    files = open_model_files(folder)
    try:
        where = {}
        for f in files:
            for name in f.names():
                if name in where:
                    raise WeightsError(f"tensor {name!r} occurs in both {where[name].path.name} and {f.path.name}")
                where[name] = f
        expected, optional = model.expected_weights()
        check_names_and_shapes({n: f.shape(n) for n, f in where.items()}, expected, optional)
        on_cpu = model.runtime.device.type == "cpu"       # a view of the mapping must not outlive it

        def fetch(name):
            t = stored_tensor(where[name], name)
            return t.clone() if on_cpu else t

        model.bind(fetch)
    finally:
        for f in files:
            f.close()
    return model
