"""Shared helpers of the engine tests: load a tiny model both ways, replay requests under
different cuts, compare with the plain implementation."""
from __future__ import annotations

import torch

import plain_llama
import tiny_models

# Bounds on |engine logit - plain logit| for the tiny models, whose logit rows have an rms of 0.2 to 0.5.
# float32: both sides compute in float32 and differ in summation order only.
# bfloat16: both sides read the same bfloat16 weights; the engine rounds activations to
# bfloat16 (8 significand bits) between parts.
# The worst values seen over the whole suite on a B200 (printed at the end of every GPU run) are
# 3.0e-6 and 1.2e-2; the bounds are about three times that.  REL_RMS bounds a row's rms error over the
# row's rms (seen: 1.8e-6 and 6.5e-3).  A greedy token is accepted when it is the plain arg-max or lies
# within TOL of it (each of the two logits may be off by half of that).
TOL = {torch.float32: 1e-5, torch.bfloat16: 3e-2}
REL_RMS = {torch.float32: 6e-6, torch.bfloat16: 1.5e-2}


def load_pair(tmp_path, which, dtype, seed=0):
    """(engine model, plain config dict, plain weights).  The folder is written in ``dtype`` so
    both sides read the same numbers."""
    from dotllm_b200 import Model
    folder = tiny_models.make_folder(tmp_path, which, seed=seed, dtype=dtype)
    cfg, weights = plain_llama.read_model_folder(folder)
    return Model.load(folder, dtype=dtype), cfg, weights, folder


# Worst errors seen by assert_close in this session, per dtype: (max |diff| / rms of the reference
# row, relative rms error of a row, max |diff|).  Printed at the end of a GPU run (conftest.py).
OBSERVED = {}


def _record(got, want, dtype):
    g, w = got.float().cpu().reshape(-1, got.shape[-1]), want.float().cpu().reshape(-1, want.shape[-1])
    rms = w.pow(2).mean(dim=-1).sqrt().clamp_min(1e-30)
    d = (g - w)
    seen = OBSERVED.setdefault(dtype, [0.0, 0.0, 0.0])
    seen[0] = max(seen[0], float((d.abs().amax(dim=-1) / rms).max()))
    seen[1] = max(seen[1], float((d.pow(2).mean(dim=-1).sqrt() / rms).max()))
    seen[2] = max(seen[2], float(d.abs().max()))


def max_err(a, b):
    return float((a.float().cpu() - b.float().cpu()).abs().max())


def assert_close(got, want, dtype, what=""):
    err = max_err(got, want)
    _record(got, want, dtype)
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    assert err <= TOL[dtype], f"{what}: max |diff| {err:.3e} > {TOL[dtype]:.1e}"
    g, w = got.float().cpu().reshape(-1, got.shape[-1]), want.float().cpu().reshape(-1, want.shape[-1])
    rel = float(((g - w).pow(2).mean(dim=-1).sqrt() / w.pow(2).mean(dim=-1).sqrt().clamp_min(1e-30)).max())
    assert rel <= REL_RMS[dtype], f"{what}: rms error of a row is {rel:.3e} of the row's rms > {REL_RMS[dtype]:.1e}"


def greedy_ok(row, token, dtype):
    """Is ``token`` an acceptable greedy choice for the plain logits ``row``: the arg-max, or within
    the bound of it (which can only be when the plain top two are closer than the bound)."""
    return int(row.argmax()) == int(token) or float(row.max() - row[token]) <= TOL[dtype]


def first_wrong(got, want, dtype):
    """Index of the first row beyond tolerance (to report where a cut goes wrong)."""
    _record(got, want, dtype)
    err = (got.float().cpu() - want.float().cpu()).abs().amax(dim=-1)
    g, w = got.float().cpu().reshape(-1, got.shape[-1]), want.float().cpu().reshape(-1, want.shape[-1])
    rel = (g - w).pow(2).mean(dim=-1).sqrt() / w.pow(2).mean(dim=-1).sqrt().clamp_min(1e-30)
    bad = ((err.reshape(-1) > TOL[dtype]) | (rel > REL_RMS[dtype])).nonzero()
    return None if bad.numel() == 0 else int(bad[0])


def penalty_history_check(device, steps=40):
    """Greedy requests with repetition penalties through ``sample_rows`` step by step, as the generation
    loop calls it - rows that end early, a window, a request without a penalty, a row whose list is
    replaced by the caller - against the plain penalty and arg-max on each step's own copy of the logits."""
    from dotllm_b200.sampling import InferenceOptions, SamplerPipeline
    from dotllm_b200.sampling.pipeline import sample_rows
    vocab = 97
    g = torch.Generator().manual_seed(5)
    options = [InferenceOptions(temperature=0.0, repetition_penalty=1.3), InferenceOptions(temperature=0.0, repetition_penalty=2.5,
               repetition_penalty_window=4), InferenceOptions(temperature=0.0), InferenceOptions(temperature=0.0, repetition_penalty=0.7),
               InferenceOptions(temperature=0.0, repetition_penalty=1.1)]
    pipes = [SamplerPipeline(o) for o in options]
    generated = [[] for _ in pipes]
    live = list(range(len(pipes)))
    for step in range(steps):
        if step == 7:
            live.remove(1)                                       # a request ends: the rows above it move down
        if step == 12:
            generated[3] = [5, 5, 9]                            # not what the device row holds: written again as a whole
        if step == 20:
            live.remove(0)
        base = (torch.randn(len(live), vocab, generator=g) * 2).round() / 2 + torch.linspace(0.3, 0, vocab)   # few distinct values: the penalty decides
        want = []
        for row, i in enumerate(live):
            o = options[i]
            x = plain_llama.apply_repetition_penalty(base[row].clone(), generated[i], o.repetition_penalty, o.repetition_penalty_window)
            want.append(int(torch.argmax(x)))
        got = sample_rows(base.clone().to(device), [pipes[i] for i in live], [generated[i] for i in live], live,
                          [len(generated[i]) for i in live])
        got = [int(t) for t in (got.tolist() if hasattr(got, "tolist") else got)]
        assert got == want, (step, got, want)
        for i, t in zip(live, got):
            generated[i].append(t)
    history = pipes[2].history
    assert history is not None and all(p.history is history for p in pipes)       # one history for the batch
    assert history.held[pipes[4].history_row] == generated[4][:-1]             # the newest id goes up with the next step
