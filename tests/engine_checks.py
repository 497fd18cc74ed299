"""Shared helpers of the engine tests: load a tiny model both ways, replay requests under
different cuts, compare with the plain implementation."""
from __future__ import annotations

import torch

import plain_llama
import tiny_models

# Bounds on |engine logit - plain logit|.  Logits of the tiny models are O(1).
# float32: both sides compute in float32 and differ in summation order only.
# bfloat16: both sides read the same bfloat16 weights; the engine rounds activations to
# bfloat16 (8 significand bits, relative step 2^-8) between parts.
TOL = {torch.float32: 2e-5, torch.bfloat16: 4e-2}


def load_pair(tmp_path, which, dtype, seed=0):
    """(engine model, plain config dict, plain weights).  The folder is written in ``dtype`` so
    both sides read the same numbers."""
    from dotllm_b200 import Model
    folder = tiny_models.make_folder(tmp_path, which, seed=seed, dtype=dtype)
    cfg, weights = plain_llama.read_model_folder(folder)
    return Model.load(folder, dtype=dtype), cfg, weights, folder


def max_err(a, b):
    return float((a.float().cpu() - b.float().cpu()).abs().max())


def assert_close(got, want, dtype, what=""):
    err = max_err(got, want)
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    assert err <= TOL[dtype], f"{what}: max |diff| {err:.3e} > {TOL[dtype]:.1e}"


def first_wrong(got, want, dtype):
    """Index of the first row beyond tolerance (to report where a cut goes wrong)."""
    err = (got.float().cpu() - want.float().cpu()).abs().amax(dim=-1)
    bad = (err > TOL[dtype]).nonzero()
    return None if bad.numel() == 0 else int(bad[0])
