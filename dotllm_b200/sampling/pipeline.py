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

    def row_temperature(self):
        """What the kernel gets: <= 0 means argmax.  In an explicit chain a temperature <= 0
        is a no-op step (TemperatureSampler.cs:25-26), i.e. T = 1."""
        if self.greedy:
            return 0.0
        return self.temperature if self.temperature > 0 else 1.0


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
        longest = max(1, max(len(g) for g in generated))
        prev = torch.zeros((rows, longest), dtype=torch.int32)
        for r, g in enumerate(generated):
            if g:
                prev[r, :len(g)] = torch.tensor(g, dtype=torch.int32)
        meta_i = torch.tensor([[len(g) for g in generated], [p.penalty_window for p in pipelines]],
                              dtype=torch.int32)
        pen = torch.tensor([p.penalty for p in pipelines], dtype=torch.float32)
        prev, meta_i, pen = prev.to(device), meta_i.to(device), pen.to(device)
        ops.repetition_penalty(logits, prev, meta_i[0].contiguous(), pen, meta_i[1].contiguous())
    for r, pipe in enumerate(pipelines):
        for step in pipe.custom_steps:
            step.apply(logits[r], pipe.context)
    if all(p.row_temperature() <= 0 for p in pipelines):
        return ops.sample(logits)
    fl = torch.tensor([[p.row_temperature() for p in pipelines],
                       [p.top_p for p in pipelines],
                       [p.min_p for p in pipelines],
                       [uniform(p.seed, n) for p, n in zip(pipelines, steps)]],
                      dtype=torch.float32).to(device)
    top_k = torch.tensor([p.top_k for p in pipelines], dtype=torch.int32).to(device)
    return ops.sample(logits, temperature=fl[0].contiguous(), top_k=top_k, top_p=fl[1].contiguous(),
                      min_p=fl[2].contiguous(), uniform=fl[3].contiguous())
