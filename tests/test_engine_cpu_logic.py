"""The engine's host logic (step planning, paged addressing, block wiring, replay) on the CPU,
with the plain kernel references standing in for the CUDA kernels."""
import io
import json

import pytest
import torch

import plain_llama
import tiny_models
from dotllm_b200.config import build_spec, load_config
from dotllm_b200.engine import StepEntry, run_step
from dotllm_b200.engine.trace import TraceReplayer
from dotllm_b200.errors import CacheFullError, StepError
from dotllm_b200.models.decoder import DecoderModel
from dotllm_b200.parts.base import Runtime
from dotllm_b200.weights import load_into

CPU = Runtime(torch.float32, torch.device("cpu"))


def load(tmp_path, which):
    folder = tiny_models.make_folder(tmp_path, which)
    cfg, weights = plain_llama.read_model_folder(folder)
    model = load_into(DecoderModel(build_spec(load_config(folder)), CPU), folder)
    return model, cfg, weights


@pytest.mark.parametrize("which", ["A", "B"])
def test_step_cuts_agree_with_the_plain_implementation(cpu_kernels, tmp_path, which):
    model, cfg, w = load(tmp_path, which)
    a = tiny_models.random_tokens(70, cfg["vocab_size"], 1)
    b = tiny_models.random_tokens(21, cfg["vocab_size"], 2)
    ra, rb = plain_llama.forward(cfg, w, a), plain_llama.forward(cfg, w, b)
    cache = model.new_cache(64 * 3)
    cache.fill_free_pages(float("nan"))
    sa, sb = cache.open_sequence(), cache.open_sequence()
    out = run_step(model, cache, [StepEntry(sa, a[:60], [0, 59]), StepEntry(sb, b[:5], [])])
    assert torch.allclose(out, ra[[0, 59]], atol=2e-5)
    for t in range(60, 70):
        entries = [StepEntry(sa, [a[t]])] + ([StepEntry(sb, [b[t - 55]])] if t - 55 < 21 else [])
        out = run_step(model, cache, entries)
        assert torch.allclose(out[0], ra[t], atol=2e-5)
        if len(entries) == 2:
            assert torch.allclose(out[1], rb[t - 55], atol=2e-5)
    assert sa.length == 70 and sb.length == 15
    cache.close_sequence(sa)
    cache.fill_free_pages(float("nan"))
    sc = cache.open_sequence()                           # reuses the slot and pages of a
    out = run_step(model, cache, [StepEntry(sc, b, None), StepEntry(sb, b[15:], None)])
    assert torch.allclose(out[0], rb[-1], atol=2e-5) and torch.allclose(out[1], rb[-1], atol=2e-5)
    cache.check()


def test_step_refuses_bad_input_before_anything_runs(cpu_kernels, tmp_path):
    model, cfg, _ = load(tmp_path, "A")
    cache = model.new_cache(128)
    s = cache.open_sequence()
    with pytest.raises(StepError, match="vocabulary"):
        run_step(model, cache, [StepEntry(s, [1, 256])])
    with pytest.raises(StepError, match="twice"):
        run_step(model, cache, [StepEntry(s, [1]), StepEntry(s, [2])])
    with pytest.raises(StepError, match="at least one"):
        run_step(model, cache, [StepEntry(s, [])])
    with pytest.raises(StepError, match="wanted offset"):
        run_step(model, cache, [StepEntry(s, [1, 2], [2])])
    with pytest.raises(StepError, match="max positions"):
        run_step(model, cache, [StepEntry(s, [1] * 129)])
    t = cache.open_sequence()
    with pytest.raises(CacheFullError):
        run_step(model, cache, [StepEntry(s, [1] * 65), StepEntry(t, [1] * 65)])
    assert s.length == 0 and t.length == 0 and cache.groups[0].pages.n_held == 0
    cache.close_sequence(t)
    with pytest.raises(StepError, match="closed"):
        run_step(model, cache, [StepEntry(t, [1])])
    with pytest.raises(StepError):
        run_step(model, cache, [])


def test_schedule_with_a_repeated_layer_and_a_shared_cache(cpu_kernels, tmp_path):
    """The order of layers is data: layer 0 runs twice (own cache each time), and a last execution
    of layer 1 reads the cache of the first execution of layer 1."""
    from dataclasses import replace
    from dotllm_b200.config.spec import ScheduleEntry
    folder = tiny_models.make_folder(tmp_path, "A")
    cfg, w = plain_llama.read_model_folder(folder)
    spec = build_spec(load_config(folder))
    spec = replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=1)))
    model = load_into(DecoderModel(spec, CPU), folder)
    cache = model.new_cache(256)
    assert len(cache.groups) == 1 and len(cache.groups[0].entries) == 3
    toks = tiny_models.random_tokens(20, 256, 4)

    def plain(tokens):
        """The same schedule written out with the plain parts."""
        n = len(tokens)
        cos, sin = plain_llama.rope_tables(range(n), 16, 10000.0)
        h = plain_llama.embed(w["model.embed_tokens.weight"], tokens)
        kept = {}
        for e, (layer, share) in enumerate([(0, None), (1, None), (0, None), (1, 1)]):
            p = f"model.layers.{layer}."
            x = plain_llama.rms_norm(h, w[p + "input_layernorm.weight"], 1e-5)
            q = plain_llama.apply_rope(plain_llama.linear(x, w[p + "self_attn.q_proj.weight"]).view(n, 4, 16), cos, sin)
            if share is None:
                k = plain_llama.apply_rope(plain_llama.linear(x, w[p + "self_attn.k_proj.weight"]).view(n, 2, 16), cos, sin)
                v = plain_llama.linear(x, w[p + "self_attn.v_proj.weight"])
                kept[e] = (k, v)
            else:
                k, v = kept[share]
            a = plain_llama.causal_attention(q.reshape(n, 64), k.reshape(n, 32), v, 4, 2, 0.25)
            h = h + plain_llama.linear(a, w[p + "self_attn.o_proj.weight"])
            x = plain_llama.rms_norm(h, w[p + "post_attention_layernorm.weight"], 1e-5)
            h = h + plain_llama.feed_forward_part(x, w, p)
        h = plain_llama.rms_norm(h, w["model.norm.weight"], 1e-5)
        return plain_llama.linear(h, w["model.embed_tokens.weight"])

    ref = plain(toks)
    s = cache.open_sequence()
    out = [run_step(model, cache, [StepEntry(s, toks[:12], list(range(12)))])]
    out += [run_step(model, cache, [StepEntry(s, [t])]) for t in toks[12:]]
    assert torch.allclose(torch.cat(out), ref, atol=2e-5)


def test_trace_replay_protocol(cpu_kernels, tmp_path):
    model, cfg, w = load(tmp_path, "A")

    class Facade:                                        # what TraceReplayer needs of a Model
        def new_cache(self, max_tokens):
            return model.new_cache(max_tokens)

        def step(self, cache, entries):
            return run_step(model, cache, entries)

    a = tiny_models.random_tokens(40, 256, 5)
    b = tiny_models.random_tokens(9, 256, 6)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:38], "want": [0, 37]},
                                     {"id": "b", "tokens": b[:8], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[38]], "want": [0]},
                                     {"id": "b", "tokens": [b[8]], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[39]], "want": []}], "end": ["a"]},
             {"step": 7, "entries": [{"id": "c", "tokens": b, "want": [8]}], "end": ["c"]}]
    out_dir = tmp_path / "out"
    replayer = TraceReplayer(Facade(), 128, out_dir)
    printed = io.StringIO()
    replayer.run([json.dumps(s) for s in steps], out=printed)
    assert printed.getvalue().split() == ["done", "0", "done", "1", "done", "2", "done", "7"]
    ra, rb = plain_llama.forward(cfg, w, a), plain_llama.forward(cfg, w, b)
    import numpy as np
    got0 = np.fromfile(out_dir / "0.f32", dtype="<f4").reshape(2, 256)
    got1 = np.fromfile(out_dir / "1.f32", dtype="<f4").reshape(2, 256)
    got7 = np.fromfile(out_dir / "7.f32", dtype="<f4").reshape(1, 256)
    assert not (out_dir / "2.f32").exists()              # nothing wanted, nothing written
    assert np.allclose(got0, ra[[0, 37]].numpy(), atol=2e-5)
    assert np.allclose(got1, torch.stack([ra[38], rb[8]]).numpy(), atol=2e-5)
    assert np.allclose(got7, rb[8:9].numpy(), atol=2e-5)
    replayer.cache.check()
    assert replayer.cache.slots.n_held == 0
    with pytest.raises(CacheFullError):                  # 4 pages asked of a 2-page cache
        replayer.run_step({"step": 9, "entries": [{"id": "x", "tokens": [1] * 100, "want": []},
                                                  {"id": "y", "tokens": [1] * 100, "want": []}], "end": []})
    assert replayer.cache.slots.n_held == 0              # the refused request holds nothing
