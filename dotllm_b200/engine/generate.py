"""The generation loop: batches of unequal prompts, one token per live sequence per step, stop
tokens, sequences that end early, and one batch after another until every request is served.

Per sequence the rules are the reference's ``TextGenerator.Generate``
(src/DotLLM.Engine/TextGenerator.cs:68-405): an empty prompt becomes [BOS] (:79-83);
``max_tokens <= 0`` yields nothing with reason "length" (:86-96); the first token is sampled from
the last prompt position's logits (:198-205); token n+1 comes from a step over token n (:347-355);
generation also ends with "length" when the next position would pass the model's positions
(:345-349); stop conditions are checked after each token is appended, first non-continue wins
(:248-262, 904-915); sampling sees the generated ids only, not the prompt (:160).

The loop itself decides nothing about kernels: it is given a step function and a sampling
function, so its decisions can be tested with stand-ins.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Optional

from ..cache.model_cache import PAGE
from ..errors import CacheFullError, StepError
from ..sampling.options import InferenceOptions
from ..sampling.pipeline import SamplerPipeline
from ..sampling.stop import (EosStopCondition, FinishReason, MaxTokensStopCondition, StopResult,
                             check_stop_conditions)
from .step import StepEntry


@dataclass
class InferenceTimings:
    """src/DotLLM.Engine/InferenceTimings.cs:6-54.  Times are those of the batch the request
    ran in; token counts are the request's own."""
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    sampling_ms: float = 0.0
    prefill_tokens: int = 0
    decode_steps: int = 0           # generated - 1 (TextGenerator.cs:1001)
    batch_size: int = 1
    batch_prefill_tokens: int = 0

    @property
    def prefill_tokens_per_sec(self):
        return self.batch_prefill_tokens / (self.prefill_ms / 1000.0) if self.prefill_ms > 0 else 0.0

    @property
    def decode_tokens_per_sec(self):
        return self.decode_steps / (self.decode_ms / 1000.0) if self.decode_ms > 0 else 0.0


@dataclass
class InferenceResponse:
    """src/DotLLM.Engine/InferenceResponse.cs:8-33, with token ids where the reference has text."""
    generated_token_ids: list
    finish_reason: FinishReason
    prompt_token_count: int
    generated_token_count: int
    timings: InferenceTimings = field(default_factory=InferenceTimings)


@dataclass
class _Request:
    index: int
    prompt: list
    options: InferenceOptions
    pipeline: SamplerPipeline
    conditions: list
    generated: list = field(default_factory=list)
    sequence: object = None
    finish_reason: Optional[FinishReason] = None
    decode_ms: float = 0.0

    def tokens_reserved(self, max_positions):
        """Worst-case cached tokens, rounded up to whole pages."""
        n = min(len(self.prompt) + max(self.options.max_tokens, 1), max_positions)
        return (n + PAGE - 1) // PAGE * PAGE


def plan_batches(requests, cache_tokens, max_batch, max_positions):
    """Cut the request list, in order, into batches whose worst-case token need fits the cache."""
    batches, current, used = [], [], 0
    for r in requests:
        need = r.tokens_reserved(max_positions)
        if need > cache_tokens:
            raise CacheFullError(f"request {r.index} may hold {need} tokens; the cache holds {cache_tokens}")
        if current and (used + need > cache_tokens or len(current) >= max_batch):
            batches.append(current)
            current, used = [], 0
        current.append(r)
        used += need
    if current:
        batches.append(current)
    return batches


class HostClock:
    """Marks are host times: right for step and sampling functions that return when their work is done."""

    def mark(self):
        return time.perf_counter()

    @staticmethod
    def ms(a, b):
        return (b - a) * 1e3


class TextGenerator:
    """Drives a step function over batches of requests.

    ``step_fn(entries) -> logits``: rows in entry order, one per entry (the last token's).
    ``sample_fn(logits, pipelines, generated, sequence_indices, steps) -> ids`` (host ints or a
    tensor).  ``cache`` opens and closes sequences and says how many tokens it can hold.
    ``fetch(ids) -> list of ints`` brings a step's sampled ids to the host; it is the one point of a
    step where the host waits for the device (the default takes ids that are already host values).
    ``clock`` marks the boundaries between a step's forward pass and its sampling for the timings:
    ``clock.mark()`` now, ``clock.ms(a, b)`` once the batch is over (so marks may be device events).

    ``ahead_fn(sequences, ids, rows) -> logits or None`` (optional) starts the next decode step
    before the host has seen this step's tokens: the step of ``sequences`` whose tokens are
    ``ids[rows]``, the sampling function's result as it is (on the device, where the model is).
    The loop calls it between ``fetch.start(ids)`` and ``fetch.finish(...)``, so that the device
    runs the next forward pass while the host waits for the ids, applies the stop rules and prepares
    the sampling.  It gives it every request that goes on unless its new token is a stop token; a
    request that then does stop has run one row in vain (rows do not depend on one another, and its
    sequence is closed right after).  None: not now; the loop then steps in the ordinary way.
    ``take_rows(logits, keep)`` picks the rows of the requests that go on."""

    def __init__(self, step_fn: Callable, sample_fn: Callable, cache, *, max_positions, vocab_size,
                 default_stop_ids=(), bos_token_id=None, max_batch=None, fetch=None, clock=None,
                 ahead_fn=None, take_rows=None):
        self.step_fn = step_fn
        self.sample_fn = sample_fn
        self.cache = cache
        self.max_positions = max_positions
        self.vocab_size = vocab_size
        self.default_stop_ids = tuple(default_stop_ids)
        self.bos_token_id = bos_token_id
        self.max_batch = max_batch or cache.n_slots
        self.fetch = fetch or (lambda ids: [int(t) for t in (ids.tolist() if hasattr(ids, "tolist") else ids)])
        self.clock = clock or HostClock()
        self.ahead_fn = ahead_fn
        self.take_rows = take_rows or (lambda logits, keep: logits[keep])
        self.ahead_steps = 0                                 # decode steps started before their tokens reached the host
        self.ahead_rows_in_vain = 0                          # rows of such steps whose request had just stopped

    # ---------------------------------------------------------------- api
    def generate(self, prompts, options=None, on_token=None):
        """``prompts``: a list of token-id lists (or one list of ints).  ``options``: one
        InferenceOptions for all, or one per prompt.  ``on_token(request_index, token_id)`` is
        called for every kept token as it is generated.  Returns one InferenceResponse per
        prompt, in order."""
        single = bool(prompts) and isinstance(prompts[0], int)
        if single:
            prompts = [prompts]
        if options is None:
            options = InferenceOptions()
        opts = list(options) if isinstance(options, (list, tuple)) else [options] * len(prompts)
        if len(opts) != len(prompts):
            raise ValueError("give one InferenceOptions, or one per prompt")
        requests = []
        responses = [None] * len(prompts)
        for i, (prompt, o) in enumerate(zip(prompts, opts)):
            prompt = [int(t) for t in prompt]
            if not prompt:
                if self.bos_token_id is None:
                    raise StepError(f"prompt {i} is empty and the model names no BOS token")
                prompt = [self.bos_token_id]
            for t in prompt:
                if not 0 <= t < self.vocab_size:
                    raise StepError(f"prompt {i}: token id {t} is outside the vocabulary [0, {self.vocab_size})")
            if len(prompt) > self.max_positions:
                raise StepError(f"prompt {i} has {len(prompt)} tokens; the model has {self.max_positions} positions")
            if o.max_tokens <= 0:
                responses[i] = InferenceResponse([], FinishReason.LENGTH, len(prompt), 0)
                continue
            if o.stop_conditions is not None:
                conditions = list(o.stop_conditions)
            else:
                stop_ids = self.default_stop_ids if o.stop_token_ids is None else tuple(o.stop_token_ids)
                conditions = ([EosStopCondition(stop_ids)] if stop_ids else []) + \
                    [MaxTokensStopCondition(o.max_tokens)]
            requests.append(_Request(i, prompt, o, SamplerPipeline(o), conditions))
        for batch in plan_batches(requests, self.cache.max_tokens, self.max_batch, self.max_positions):
            self._run_batch(batch, on_token)
            for r in batch:
                responses[r.index] = r.response
        return responses[0] if single else responses

    # -------------------------------------------------------------- a batch
    def _finish(self, r, reason):
        r.finish_reason = reason
        if r.sequence is not None and r.sequence.open:
            self.cache.close_sequence(r.sequence)           # the slot and pages are free for the next batch

    def _accept(self, r, token, on_token):
        """Append a sampled token and apply the stop rules.  True if the request goes on."""
        r.generated.append(token)
        verdict = check_stop_conditions(r.conditions, token, r.generated)
        if verdict == StopResult.STOP:
            r.generated.pop()                               # EosStopCondition.cs:23-24
            self._finish(r, FinishReason.STOP)
            return False
        if on_token is not None:
            on_token(r.index, token)
        if verdict == StopResult.STOP_INCLUDE:
            self._finish(r, FinishReason.LENGTH)
            return False
        if self._last_token(r, len(r.generated)):
            self._finish(r, FinishReason.LENGTH)
            return False
        return True

    def _last_token(self, r, n_generated):
        """Is the request's token number ``n_generated`` its last, whatever it is?  (A caller's own
        conditions may lack the cap; the next step would place the token at position
        prompt + generated - 1.)"""
        return n_generated >= r.options.max_tokens or len(r.prompt) + n_generated - 1 >= self.max_positions

    def _sample(self, logits, live):
        return self.sample_fn(logits, [r.pipeline for r in live], [r.generated for r in live],
                              [r.index for r in live], [len(r.generated) for r in live])

    def _step_ahead(self, live, ids):
        """Start the next decode step for the requests that go on unless their new token stops them.
        Returns (those requests, logits, marks around the forward pass), or None."""
        rows = [i for i, r in enumerate(live) if not self._last_token(r, len(r.generated) + 1)]
        if not rows:
            return None
        t0 = self.clock.mark()
        logits = self.ahead_fn([live[i].sequence for i in rows], ids, rows)
        if logits is None:
            return None
        self.ahead_steps += 1
        return [live[i] for i in rows], logits, t0, self.clock.mark()

    def _run_batch(self, batch, on_token):
        clock = self.clock
        marks = []                                           # per step: before the forward pass, after it, after sampling
        try:
            for r in batch:
                r.sequence = self.cache.open_sequence()
            t0 = clock.mark()
            logits = self.step_fn([StepEntry(r.sequence, r.prompt) for r in batch])
            t1 = clock.mark()
            ids = self._sample(logits, batch)
            t2 = clock.mark()
            marks.append((t0, t1, t1, t2, None))
            live = batch
            while True:
                start = getattr(self.fetch, "start", None)
                pending = start(ids) if start is not None else None
                ahead = self._step_ahead(live, ids) if self.ahead_fn is not None else None
                tokens = self.fetch.finish(pending) if start is not None else self.fetch(ids)   # the step's one wait for the device
                live = [r for r, tok in zip(live, tokens) if self._accept(r, tok, on_token)]
                if not live:
                    break
                if ahead is not None:
                    ran, logits, t0, t1 = ahead
                    if len(ran) != len(live):
                        going = {id(r) for r in live}
                        keep = [i for i, r in enumerate(ran) if id(r) in going]
                        self.ahead_rows_in_vain += len(ran) - len(keep)
                        if len(keep) != len(live):
                            raise RuntimeError("a request goes on that the step started ahead did not hold")
                        logits = self.take_rows(logits, keep)
                else:
                    t0 = clock.mark()
                    logits = self.step_fn([StepEntry(r.sequence, [r.generated[-1]]) for r in live])
                    t1 = clock.mark()
                ts = clock.mark()
                ids = self._sample(logits, live)
                t2 = clock.mark()
                marks.append((t0, t1, ts, t2, list(live)))
        finally:
            for r in batch:                                  # an error must not leak slots
                if r.sequence is not None and r.sequence.open:
                    self.cache.close_sequence(r.sequence)
        prefill_ms = clock.ms(marks[0][0], marks[0][1])
        sampling_ms = sum(clock.ms(ts, t2) for _, _, ts, t2, _ in marks)
        for t0, t1, _, _, live in marks[1:]:
            step_ms = clock.ms(t0, t1)
            for r in live:
                r.decode_ms += step_ms
        total_prompt = sum(len(r.prompt) for r in batch)
        for r in batch:
            r.response = InferenceResponse(
                list(r.generated), r.finish_reason, len(r.prompt), len(r.generated),
                InferenceTimings(prefill_ms=prefill_ms, decode_ms=r.decode_ms,
                                 sampling_ms=sampling_ms, prefill_tokens=len(r.prompt),
                                 decode_steps=max(0, len(r.generated) - 1), batch_size=len(batch),
                                 batch_prefill_tokens=total_prompt))
