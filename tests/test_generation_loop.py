"""The generation loop's decisions, with a scripted model in place of the kernels."""
import pytest
import torch

from dotllm_b200.cache import ModelCache
from dotllm_b200.engine import TextGenerator, plan_batches
from dotllm_b200.errors import CacheFullError, StepError
from dotllm_b200.parts.base import CacheNeed, Runtime
from dotllm_b200.sampling import (EosStopCondition, FinishReason, InferenceOptions, MaxTokensStopCondition,
                                  SamplerPipeline, StopCondition, StopResult, TemperatureSampler,
                                  TopKSampler, uniform)

CPU = Runtime(torch.float32, torch.device("cpu"))
VOCAB = 50


class ScriptedModel:
    """Next token = (last token + 1) % VOCAB.  Records every step it is asked to run."""

    def __init__(self, cache):
        self.cache = cache
        self.steps = []

    def step(self, entries):
        self.steps.append([(e.sequence.slot, list(e.tokens), e.sequence.length) for e in entries])
        self.cache.reserve([(e.sequence, e.sequence.length + len(e.tokens)) for e in entries])
        for e in entries:
            self.cache.commit(e.sequence, e.sequence.length + len(e.tokens))
        logits = torch.zeros(len(entries), VOCAB)
        for i, e in enumerate(entries):
            logits[i, (e.tokens[-1] + 1) % VOCAB] = 5.0
        return logits

    @staticmethod
    def sample(logits, pipelines, generated, seq_indices, steps):
        return [int(t) for t in logits.argmax(dim=-1)]


def make(max_tokens=64 * 8, max_positions=128, stop=(), bos=None, max_batch=None, slots=None):
    cache = ModelCache([CacheNeed("kv", n_kv_heads=1, head_dim=16)], [None], CPU, max_tokens, slots)
    model = ScriptedModel(cache)
    gen = TextGenerator(model.step, model.sample, cache, max_positions=max_positions, vocab_size=VOCAB,
                        default_stop_ids=stop, bos_token_id=bos, max_batch=max_batch)
    return gen, model, cache


GREEDY = dict(temperature=0.0)


def test_prompts_in_one_step_then_one_token_each():
    gen, model, cache = make()
    outs = gen.generate([[3, 4, 5], [10], [20, 21]], InferenceOptions(max_tokens=4, **GREEDY))
    assert [o.generated_token_ids for o in outs] == [[6, 7, 8, 9], [11, 12, 13, 14], [22, 23, 24, 25]]
    assert all(o.finish_reason == FinishReason.LENGTH for o in outs)
    assert [len(s) for s in model.steps] == [3, 3, 3, 3]            # one prefill, three decode steps
    assert [e[1] for e in model.steps[0]] == [[3, 4, 5], [10], [20, 21]]
    assert [e[1] for e in model.steps[1]] == [[6], [11], [22]]      # the token just generated
    assert [e[2] for e in model.steps[1]] == [3, 1, 2]              # continuing from each one's own length
    assert outs[0].timings.decode_steps == 3 and outs[0].prompt_token_count == 3
    cache.check()
    assert cache.slots.n_held == 0


def test_stop_token_is_dropped_and_ends_only_its_own_request():
    gen, model, cache = make(stop=(13,))
    outs = gen.generate([[3], [10], [40]], InferenceOptions(max_tokens=6, **GREEDY))
    assert outs[1].generated_token_ids == [11, 12] and outs[1].finish_reason == FinishReason.STOP
    assert outs[0].generated_token_ids == [4, 5, 6, 7, 8, 9] and outs[0].finish_reason == FinishReason.LENGTH
    assert [len(s) for s in model.steps] == [3, 3, 3, 2, 2, 2]      # the stopped one left the batch
    stopped_slot = model.steps[0][1][0]
    assert all(e[0] != stopped_slot for s in model.steps[3:] for e in s)
    per_request = gen.generate([[10]], InferenceOptions(max_tokens=6, stop_token_ids=[], **GREEDY))
    assert per_request[0].generated_token_ids == [11, 12, 13, 14, 15, 16]     # an empty set disables stops
    first_is_stop = gen.generate([[12]], InferenceOptions(max_tokens=6, **GREEDY))
    assert first_is_stop[0].generated_token_ids == [] and first_is_stop[0].finish_reason == FinishReason.STOP


def test_max_tokens_and_empty_cases():
    gen, model, _ = make(bos=1)
    outs = gen.generate([[5], [6]], [InferenceOptions(max_tokens=0, **GREEDY), InferenceOptions(max_tokens=1, **GREEDY)])
    assert outs[0].generated_token_ids == [] and outs[0].finish_reason == FinishReason.LENGTH
    assert outs[1].generated_token_ids == [7] and len(model.steps) == 1
    assert gen.generate([[]], InferenceOptions(max_tokens=2, **GREEDY))[0].generated_token_ids == [2, 3]   # [BOS]
    single = gen.generate([7, 8], InferenceOptions(max_tokens=2, **GREEDY))
    assert single.generated_token_ids == [9, 10]                    # one prompt in, one response out
    gen2, _, _ = make()
    with pytest.raises(StepError, match="BOS"):
        gen2.generate([[]], InferenceOptions(max_tokens=2, **GREEDY))
    with pytest.raises(StepError, match="vocabulary"):
        gen2.generate([[VOCAB]], InferenceOptions(max_tokens=2, **GREEDY))


def test_generation_ends_at_the_models_last_position():
    gen, model, _ = make(max_positions=8)
    out = gen.generate([[1, 2, 3, 4, 5]], InferenceOptions(max_tokens=50, **GREEDY))[0]
    # positions 0..7: 5 prompt tokens, decode steps at positions 5, 6, 7 -> 1 + 3 tokens
    assert out.generated_token_ids == [6, 7, 8, 9] and out.finish_reason == FinishReason.LENGTH
    assert model.steps[-1][0][2] == 7
    with pytest.raises(StepError, match="positions"):
        gen.generate([[1] * 9], InferenceOptions(max_tokens=1, **GREEDY))


def test_batches_follow_one_another_and_reuse_slots():
    gen, model, cache = make(max_tokens=64 * 2, slots=2)
    prompts = [[i] for i in range(5)]
    outs = gen.generate(prompts, InferenceOptions(max_tokens=3, **GREEDY))
    assert [o.generated_token_ids for o in outs] == [[i + 1, i + 2, i + 3] for i in range(5)]
    sizes = [len(s) for s in model.steps]
    assert sizes == [2, 2, 2, 2, 2, 2, 1, 1, 1]                     # 2 + 2 + 1 requests
    slots_used = {e[0] for s in model.steps for e in s}
    assert slots_used == {0, 1}
    cache.check()
    assert cache.groups[0].pages.n_held == 0
    gen3, model3, _ = make(max_batch=3)
    gen3.generate(prompts, InferenceOptions(max_tokens=1, **GREEDY))
    assert [len(s) for s in model3.steps] == [3, 2]


def test_plan_batches_by_worst_case_tokens():
    gen, _, _ = make(max_tokens=64 * 4, max_positions=1000)
    with pytest.raises(CacheFullError):
        gen.generate([[1] * 100], InferenceOptions(max_tokens=200, **GREEDY))    # 300 tokens > 256

    class R:
        def __init__(self, i, n):
            self.index, self.n = i, n

        def tokens_reserved(self, max_positions):
            return self.n
    batches = plan_batches([R(0, 128), R(1, 128), R(2, 64), R(3, 256)], 256, 10, 1000)
    assert [[r.index for r in b] for b in batches] == [[0, 1], [2], [3]]


def test_an_error_in_a_step_leaks_no_slot():
    gen, model, cache = make()
    calls = {"n": 0}
    real = model.step

    def failing(entries):
        calls["n"] += 1
        if calls["n"] == 2:
            raise RuntimeError("boom")
        return real(entries)
    gen.step_fn = failing
    with pytest.raises(RuntimeError):
        gen.generate([[1], [2]], InferenceOptions(max_tokens=5, **GREEDY))
    cache.check()
    assert cache.slots.n_held == 0 and cache.groups[0].pages.n_held == 0


def test_custom_stop_conditions_and_callback():
    class StopAtSeven(StopCondition):
        def should_stop(self, token_id, generated):
            return StopResult.STOP_INCLUDE if token_id == 7 else StopResult.CONTINUE
    gen, _, _ = make()
    seen = []
    out = gen.generate([[4]], InferenceOptions(max_tokens=10, stop_conditions=[StopAtSeven()], **GREEDY),
                       on_token=lambda i, t: seen.append((i, t)))[0]
    assert out.generated_token_ids == [5, 6, 7] and out.finish_reason == FinishReason.LENGTH
    assert seen == [(0, 5), (0, 6), (0, 7)]
    capped = gen.generate([[20]], InferenceOptions(max_tokens=3, stop_conditions=[StopAtSeven()], **GREEDY))[0]
    assert capped.generated_token_ids == [21, 22, 23]               # the cap holds without a condition for it
    assert EosStopCondition([3]).should_stop(3, [3]) == StopResult.STOP
    assert MaxTokensStopCondition(2).should_stop(0, [1, 2]) == StopResult.STOP_INCLUDE


def test_pipeline_is_built_like_the_references():
    p = SamplerPipeline(InferenceOptions(temperature=0.0, top_k=5))
    assert p.greedy and p.row_temperature() == 0.0
    p = SamplerPipeline(InferenceOptions())                          # defaults: T=0.7, nothing else
    assert not p.greedy and p.temperature == pytest.approx(0.7) and p.top_k == 0 and p.top_p == 1.0 and p.penalty == 1.0
    p = SamplerPipeline(InferenceOptions(temperature=1.0, top_k=40, top_p=0.9, min_p=0.05, repetition_penalty=1.2,
                                         repetition_penalty_window=16, seed=3))
    assert (p.row_temperature(), p.top_k, p.top_p, p.min_p, p.penalty, p.penalty_window, p.seed) == \
        (1.0, 40, pytest.approx(0.9), pytest.approx(0.05), pytest.approx(1.2), 16, 3)
    p = SamplerPipeline(InferenceOptions(temperature=0.0, sampler_steps=[TopKSampler(3)]))
    assert not p.greedy and p.top_k == 3 and p.row_temperature() == 1.0      # explicit chains always draw
    with pytest.raises(ValueError, match="order"):
        SamplerPipeline(InferenceOptions(sampler_steps=[TopKSampler(3), TemperatureSampler(0.5)]))
    with pytest.raises(ValueError):
        InferenceOptions(repetition_penalty=0.0).validate()


def test_repetition_penalty_from_a_history_kept_between_steps(cpu_kernels):
    from engine_checks import penalty_history_check
    penalty_history_check(torch.device("cpu"))


def test_uniform_numbers_depend_on_seed_and_step_only():
    a = [uniform(1, s) for s in range(200)]
    assert all(0.0 <= u < 1.0 for u in a) and len(set(a)) > 190
    assert a == [uniform(1, s) for s in range(200)]
    assert uniform(1, 1) != uniform(1, 0) != uniform(2, 0)
    assert abs(sum(uniform(i, j) for i in range(50) for j in range(50)) / 2500 - 0.5) < 0.02


def test_a_device_bound_batch_size_waits_longer_for_its_graph():
    """The rule that decides when a decode batch size is captured: at once where the host's launches
    bound the step (or nothing is known yet), much later where the device does."""
    from dotllm_b200.engine.decode_graph import LAUNCH_BOUND, LAUNCH_BOUND_PATIENCE, sightings_needed
    assert sightings_needed(8, None) == 8
    assert sightings_needed(8, 1.3) == 8
    assert sightings_needed(8, LAUNCH_BOUND) == 8
    assert sightings_needed(8, 0.5) == 8 * LAUNCH_BOUND_PATIENCE
    assert sightings_needed(0, 0.5) == 0                     # graphs=True: always at once


class OrderedFetch:
    """A fetch in two halves that records when each half ran."""

    def __init__(self, log):
        self.log = log

    def start(self, ids):
        self.log.append("fetch starts")
        return list(ids)

    def finish(self, pending):
        self.log.append("fetch ends")
        return [int(t) for t in pending]


def make_ahead(refuse_first=0, **kw):
    from dotllm_b200.engine import StepEntry
    gen, model, cache = make(**kw)
    log, refused = [], [refuse_first]

    def ahead(sequences, ids, rows):
        log.append(("ahead", [s.slot for s in sequences], [ids[i] for i in rows]))
        if refused[0] > 0:
            refused[0] -= 1
            return None
        return model.step([StepEntry(s, [ids[i]]) for s, i in zip(sequences, rows)])

    gen.ahead_fn = ahead
    gen.fetch = OrderedFetch(log)
    return gen, model, cache, log


def test_steps_started_ahead_give_the_same_tokens():
    """With a function that starts the next step before the tokens are on the host, every request
    gets the tokens it gets without; the step starts between the two halves of the fetch; a request
    whose next token is its last by the count is left out of it; a request that meets its stop token
    has run one row in vain, and the others' rows are picked from the step's result."""
    prompts = [[3], [10], [40], [20, 21]]
    options = [InferenceOptions(max_tokens=n, **GREEDY) for n in (6, 6, 3, 5)]
    plain, plain_model, _ = make(stop=(13,))
    want = plain.generate(prompts, options)
    gen, model, cache, log = make_ahead(stop=(13,))
    got = gen.generate(prompts, options)
    assert [o.generated_token_ids for o in got] == [o.generated_token_ids for o in want]
    assert [o.finish_reason for o in got] == [o.finish_reason for o in want]
    assert got[1].generated_token_ids == [11, 12] and got[1].finish_reason == FinishReason.STOP
    # order within a step: the copy is sent, the next step starts, the host waits for the copy
    assert log[:3] == ["fetch starts", ("ahead", [0, 1, 2, 3], [4, 11, 41, 22]), "fetch ends"]
    sizes = [len(s) for s in model.steps]
    # prompts; 4 rows; 4 rows (request 2's third token is its last: it is left out of the step after);
    # 3 rows, of which request 1's ran in vain (its token 13 stopped it); 2; 1 (request 3 left: fifth token)
    assert sizes == [4, 4, 4, 3, 2, 1]
    assert sizes != [len(s) for s in plain_model.steps]               # [4, 4, 4, 2, 2, 1] without
    assert gen.ahead_rows_in_vain == 1 and gen.ahead_steps == 5
    assert [o.timings.decode_steps for o in got] == [5, 1, 2, 4]
    cache.check()
    assert cache.slots.n_held == 0


def test_a_refused_step_ahead_falls_back_to_the_ordinary_step():
    gen, model, cache, log = make_ahead(refuse_first=2)
    outs = gen.generate([[3], [10]], InferenceOptions(max_tokens=5, **GREEDY))
    assert [o.generated_token_ids for o in outs] == [[4, 5, 6, 7, 8], [11, 12, 13, 14, 15]]
    assert [len(s) for s in model.steps] == [2, 2, 2, 2, 2]
    assert gen.ahead_steps == 2 and sum(1 for e in log if isinstance(e, tuple)) == 4
    cache.check()


def test_steps_ahead_stop_at_the_models_last_position():
    gen, model, cache, _ = make_ahead(max_positions=8)
    out = gen.generate([[1, 2, 3, 4, 5]], InferenceOptions(max_tokens=50, **GREEDY))[0]
    assert out.generated_token_ids == [6, 7, 8, 9] and out.finish_reason == FinishReason.LENGTH
    assert model.steps[-1][0][2] == 7 and len(model.steps) == 4        # no step beyond the last position
    cache.check()


def test_widths_of_the_loops_decode_graphs():
    """A graph of `graph_rows(b)` rows serves b sequences: powers of two up to 16, multiples of 16
    above, never fewer rows than sequences, and few widths for many batch sizes."""
    from dotllm_b200.engine.decode_graph import graph_rows
    assert [graph_rows(b) for b in (1, 2, 3, 4, 5, 8, 9, 16, 17, 32, 33, 48, 49, 64, 65, 200)] == \
        [1, 2, 4, 4, 8, 8, 16, 16, 32, 32, 48, 48, 64, 64, 80, 208]
    assert all(graph_rows(b) >= b for b in range(1, 600))
    assert len({graph_rows(b) for b in range(1, 65)}) == 8
