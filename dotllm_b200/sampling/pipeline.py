"""The sampler pipeline: logit processors, then greedy argmax or the chain
temperature -> top-k -> top-p -> min-p -> categorical draw.

Shape and order follow the reference's ``SamplerPipeline``
(src/DotLLM.Engine/Samplers/SamplerPipeline.cs:55-157): processors are added only when enabled,
greedy when ``temperature <= 0``, and each step only when its option is on.  The reference runs
the chain on the host over a copy of the logits; here the built-in processors and steps are
parameters of device kernels (csrc/sampling.cu) that handle a whole batch of rows in one launch,
each row with its own options.  A caller's own ``SamplerStep`` / ``LogitProcessor`` objects
(``ISamplerStep`` / ``ILogitProcessor``, src/DotLLM.Core/Sampling/ISamplerStep.cs:8-16) get the row's
logits as a device tensor and may change them in place before the built-in chain runs.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from ..kernels import ops
from .options import InferenceOptions
from .rng import uniform


@dataclass
class SamplerContext:
    """Options a step may read (src/DotLLM.Core/Sampling/SamplerContext.cs)."""
    temperature: float
    top_k: int
    top_p: float
    min_p: float
    seed: int


class SamplerStep:
    """One step of the chain.  Built-in steps set a field of the kernel's parameters
    (``configure``); a custom step overrides ``apply`` and edits the logits row in place."""

    def configure(self, params):
        return None

    def apply(self, logits, context):
        return None


class TemperatureSampler(SamplerStep):
    """logits *= 1/T (src/DotLLM.Engine/Samplers/TemperatureSampler.cs:22-29)."""

    def __init__(self, temperature=None):
        self.temperature = temperature

    def configure(self, params):
        if self.temperature is not None:
            params["temperature"] = float(self.temperature)
        params["use_temperature"] = True


class TopKSampler(SamplerStep):
    """Keep the k largest logits (src/DotLLM.Engine/Samplers/TopKSampler.cs:32-79)."""

    def __init__(self, top_k=None):
        self.top_k = top_k

    def configure(self, params):
        if self.top_k is not None:
            params["top_k"] = int(self.top_k)
        params["use_top_k"] = True


class TopPSampler(SamplerStep):
    """Keep the smallest set of most probable tokens reaching p
    (src/DotLLM.Engine/Samplers/TopPSampler.cs:23-81)."""

    def __init__(self, top_p=None):
        self.top_p = top_p

    def configure(self, params):
        if self.top_p is not None:
            params["top_p"] = float(self.top_p)
        params["use_top_p"] = True


class MinPSampler(SamplerStep):
    """Mask logits below max + ln(min_p) (src/DotLLM.Engine/Samplers/MinPSampler.cs:23-37)."""

    def __init__(self, min_p=None):
        self.min_p = min_p

    def configure(self, params):
        if self.min_p is not None:
            params["min_p"] = float(self.min_p)
        params["use_min_p"] = True


class CategoricalSampler:
    """The final draw: first index whose running probability exceeds r
    (src/DotLLM.Engine/Samplers/CategoricalSampler.cs:18-41).  Always last; part of the kernel."""


class LogitProcessor:
    """Edits logits before sampling, given the ids generated so far
    (src/DotLLM.Core/Sampling/ILogitProcessor.cs)."""

    def configure(self, params):
        return None

    def process(self, logits, previous_tokens, context):
        return None


class RepetitionPenaltyProcessor(LogitProcessor):
    """Each distinct id among the last ``window`` generated tokens: positive logits divided by
    the penalty, others multiplied (src/DotLLM.Engine/Samplers/RepetitionPenaltyProcessor.cs:14-55)."""

    def configure(self, params):
        params["use_penalty"] = True


_BUILTIN_ORDER = (TemperatureSampler, TopKSampler, TopPSampler, MinPSampler)


class SamplerPipeline:
    """The chain of one request."""

    def __init__(self, options: InferenceOptions):
        options.validate()
        self.options = options
        self.seed = options.seed if options.seed is not None else int.from_bytes(os.urandom(8), "little")
        p = {"temperature": float(options.temperature), "top_k": int(options.top_k),
             "top_p": float(options.top_p), "min_p": float(options.min_p),
             "use_temperature": False, "use_top_k": False, "use_top_p": False, "use_min_p": False,
             "use_penalty": False}
        self.custom_steps = []
        self.custom_processors = []
        # processors (SamplerPipeline.cs:70-84, 92-105)
        if options.logit_processors is not None:
            processors = list(options.logit_processors)
        else:
            processors = [RepetitionPenaltyProcessor()] if options.repetition_penalty != 1.0 else []
        for proc in processors:
            proc.configure(p)
            if type(proc).process is not LogitProcessor.process:
                self.custom_processors.append(proc)
        # steps (SamplerPipeline.cs:59-66, 107-119)
        if options.sampler_steps is not None:
            self.greedy = False
            steps = list(options.sampler_steps)
        else:
            self.greedy = options.temperature <= 0
            steps = []
            if not self.greedy:
                if options.temperature != 1.0:
                    steps.append(TemperatureSampler())
                if options.top_k > 0:
                    steps.append(TopKSampler())
                if options.top_p < 1.0:
                    steps.append(TopPSampler())
                if options.min_p > 0:
                    steps.append(MinPSampler())
        last = -1
        for step in steps:
            if type(step).apply is not SamplerStep.apply:
                self.custom_steps.append(step)
                continue
            rank = next((i for i, c in enumerate(_BUILTIN_ORDER) if isinstance(step, c)), None)
            if rank is None:
                raise ValueError(f"{type(step).__name__} neither overrides apply() nor is a built-in step")
            if rank <= last:
                raise ValueError("built-in steps run in the order temperature, top-k, top-p, min-p, once each")
            last = rank
            step.configure(p)
        self.temperature = p["temperature"] if p["use_temperature"] else 1.0
        self.top_k = p["top_k"] if p["use_top_k"] else 0
        self.top_p = p["top_p"] if p["use_top_p"] else 1.0
        self.min_p = p["min_p"] if p["use_min_p"] else 0.0
        self.penalty = float(options.repetition_penalty) if p["use_penalty"] else 1.0
        self.penalty_window = int(options.repetition_penalty_window)
        self.context = SamplerContext(options.temperature, options.top_k, options.top_p, options.min_p, self.seed)
        self.history, self.history_row = None, -1            # the batch's PenaltyHistory and this request's row in it

    def row_temperature(self):
        """What the kernel gets: <= 0 means argmax.  In an explicit chain a temperature <= 0
        is a no-op step (TemperatureSampler.cs:25-26), i.e. T = 1."""
        if self.greedy:
            return 0.0
        return self.temperature if self.temperature > 0 else 1.0


class PenaltyHistory:
    """The ids that the requests of one batch have generated, kept on the device for the repetition
    penalty: a request's pipeline is given a row when the penalty first sees it, and every step sends
    the one new id per row (the kernel writes it into the row before it reads the row) instead of all
    ids generated so far.  A row whose request's list does not continue what the row holds (a
    caller's own list, a token taken back) is written again as a whole."""

    def __init__(self, device, rows=8, tokens=256):
        self.device = device
        self.ids = torch.zeros((rows, tokens), dtype=torch.int32, device=device)
        self.held = []                                       # per row: the ids the device row holds (host copy)

    def _grow(self, rows, tokens):
        have_r, have_t = self.ids.shape
        if rows <= have_r and tokens <= have_t:
            return
        new_r, new_t = max(have_r, rows), have_t
        while new_t < tokens:
            new_t *= 2
        if new_r > have_r:
            new_r = max(new_r, 2 * have_r)
        bigger = torch.zeros((new_r, new_t), dtype=torch.int32, device=self.device)
        bigger[:have_r, :have_t] = self.ids
        self.ids = bigger

    def row_of(self, pipe):
        if pipe.history is not self:
            pipe.history, pipe.history_row = self, len(self.held)
            self.held.append([])
        return pipe.history_row

    def step(self, pipelines, generated):
        """Bring the rows of these pipelines up to date.  Returns (row map, positions and ids to append,
        lengths) as host lists; rows that had to be rewritten are already on the device."""
        rows, pos, tok, lens = [], [], [], []
        mine = [self.row_of(pipe) for pipe in pipelines]
        self._grow(len(self.held), max((len(g) for g in generated), default=0) + 1)
        for h, g in zip(mine, generated):
            held = self.held[h]
            n = len(g)
            if n == len(held) + 1 and (n == 1 or g[-2] == held[-1]):
                pos.append(n - 1)
                tok.append(int(g[-1]))
                held.append(int(g[-1]))
            elif n == len(held) and (n == 0 or g[-1] == held[-1]):
                pos.append(-1)
                tok.append(0)
            else:                                             # not the continuation of what the row holds
                self.held[h] = [int(t) for t in g]
                if n:
                    self.ids[h, :n] = _to_device(self.held[h], torch.int32, self.device)
                pos.append(-1)
                tok.append(0)
            rows.append(h)
            lens.append(n)
        return rows, pos, tok, lens


def _to_device(values, dtype, device):
    """Host numbers to a device tensor through pinned memory, without waiting for the stream: a copy
    from pageable memory would hold the host until the step before it has finished."""
    host = torch.tensor(values, dtype=dtype, pin_memory=device.type == "cuda")
    return host.to(device, non_blocking=True)


def _penalise(logits, pipelines, generated):
    """The repetition penalty of every row, from the batch's history on the device."""
    history = next((p.history for p in pipelines if p.history is not None), None)
    if history is None or history.device != logits.device:
        history = PenaltyHistory(logits.device)
    rows, pos, tok, lens = history.step(pipelines, generated)
    meta = _to_device([rows, pos, tok, lens, [p.penalty_window for p in pipelines]], torch.int32, logits.device)
    pen = _to_device([p.penalty for p in pipelines], torch.float32, logits.device)
    ops.repetition_penalty(logits, history.ids, meta[3], pen, meta[4], row_map=meta[0], append=(meta[1], meta[2]))


def sample_rows(logits, pipelines, generated, sequence_indices, steps):
    """One token for every row of ``logits`` (float32 [R, V] on the device).

    ``pipelines[r]``, ``generated[r]`` (ids generated so far by row r's request) and ``steps[r]``
    (how many tokens it has generated) belong to row r.  A row's draw depends on its request's seed
    and step only: ``sequence_indices`` (the request's place in the caller's list) plays no part, so
    the same request gives the same tokens alone, in any batch, at any place in it.
    Returns an int32 device tensor [R]."""
    rows = logits.shape[0]
    device = logits.device
    # custom processors and steps see their row as a device tensor
    for r, pipe in enumerate(pipelines):
        for proc in pipe.custom_processors:
            proc.process(logits[r], generated[r], pipe.context)
    if any(p.penalty != 1.0 for p in pipelines):
        _penalise(logits, pipelines, generated)
    for r, pipe in enumerate(pipelines):
        for step in pipe.custom_steps:
            step.apply(logits[r], pipe.context)
    if all(p.row_temperature() <= 0 for p in pipelines):
        return ops.sample(logits)
    fl = _to_device([[p.row_temperature() for p in pipelines],
                     [p.top_p for p in pipelines],
                     [p.min_p for p in pipelines],
                     [uniform(p.seed, n) for p, n in zip(pipelines, steps)]], torch.float32, device)
    top_k = _to_device([p.top_k for p in pipelines], torch.int32, device)
    return ops.sample(logits, temperature=fl[0].contiguous(), top_k=top_k, top_p=fl[1].contiguous(),
                      min_p=fl[2].contiguous(), uniform=fl[3].contiguous())
