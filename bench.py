"""Decode and prefill throughput of the Llama-3.1-8B-shaped model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 8192] [--layers L]
                    [--dtype bfloat16|float32] [--shape 8b|1b|13b] [--repeats 5]
    python bench.py --shape 1b --workload unequal     # 64 prompts of 16..2048 tokens in one step, then 256 decode steps
    python bench.py --workload staggered              # Model.generate while 64 requests end one by one (also --shape 1b)
    python bench.py --workload short-prompts          # time to the first token of single short prompts, eager and captured
    python bench.py --impl plain-cpu                  # the plain implementation under tests/, timed on the CPU

A "step" is one decode step: one new token for each of ``batch`` sequences that already hold
``context`` tokens.  ``value`` is decoded tokens per second, timed on the device with CUDA events
over K consecutive steps (every step reads all weights, far more than the L2 holds).  ``e2e`` is
the same through the public entry point with host token ids in and out every step.  The line also
carries a 2,048-token prefill, decode at batch 1 and 64, the decode step's HBM roofline, the share
of an eager step's kernel time per kernel family, and tokens per second of ``Model.generate`` itself
(the loop users call: prompts in, 256 new tokens each out, stop tokens off).  Every timed region is
repeated ``--repeats`` times; the best repetition is reported with the coefficient of variation over
all of them (the reference's protocol, benchmarks/DotLLM.Benchmarks/InferenceBenchmarks.cs:30).

The cache contents are random numbers written directly into the pages: a decode step's time does
not depend on the values it reads, and filling 64 x 8192 positions through the model would take
longer than the whole measurement.  Weights are random (seeded), token ids synthetic.

The reference (kkokosa/dotLLM) is a .NET 10 program that loads GGUF checkpoints; neither the SDK
nor a checkpoint can be had offline here, so ``--impl reference`` reports itself unavailable.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_31_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 131072,
    "hidden_act": "silu",
}
# The other two benchmark shapes of the same architecture (selected with --shape).
LLAMA_32_1B = dict(LLAMA_31_8B, num_hidden_layers=16, hidden_size=2048, num_attention_heads=32, num_key_value_heads=8,
                   head_dim=64, intermediate_size=8192, vocab_size=128256, tie_word_embeddings=True,
                   rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                 "original_max_position_embeddings": 8192})
LLAMA_2_13B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 40, "hidden_size": 5120, "num_attention_heads": 40, "num_key_value_heads": 40,
    "head_dim": 128, "intermediate_size": 13824, "vocab_size": 32000, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 4096, "hidden_act": "silu",
}
SHAPES = {"8b": ("Llama-3.1-8B-shaped", LLAMA_31_8B), "1b": ("Llama-3.2-1B-shaped", LLAMA_32_1B),
          "13b": ("Llama-2-13B-shaped", LLAMA_2_13B)}
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
FP32_TFLOPS_NOMINAL = 74.5      # 148 multiprocessors x 128 FMA a clock x 2 x 1.965 GHz: no measured float32 peak exists


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            data = json.load(open(path))
            return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]), "source": "measured"}
        except (OSError, ValueError, KeyError):
            pass
    return {**FALLBACK_PEAKS, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples taken while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "plain-cpu"])
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--repeats", type=int, default=5, help="repetitions of every timed region (best and CV are reported)")
    ap.add_argument("--workload", default="steady", choices=["steady", "unequal", "staggered", "short-prompts"],
                    help="unequal: 64 prompts of 16..2048 tokens in one prefill step, then 256 decode steps; "
                         "staggered: Model.generate on 64 prompts whose requests end five steps apart; "
                         "short-prompts: the time to the first token of single prompts of 20 to 1,024 tokens")
    ap.add_argument("--no-generate", action="store_true", help="skip the Model.generate cells")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes: the 8B default, or 1b / 13b")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (0: all of them)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points and the prefill")
    ap.add_argument("--only-prefill", action="store_true", help="run only the 2,048-token prefill (for profiling)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="with --only-prefill: tokens of the one prompt (the line itself always reports 2,048)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference",
                          "unavailable": "kkokosa/dotLLM is a .NET 10 program reading GGUF checkpoints; no .NET SDK, "
                                         "no checkpoint and no network exist here, so it cannot be installed or run"}))
        return 0
    if args.impl == "plain-cpu":
        return plain_cpu_baseline()
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU library: --gpus {args.gpus} is not supported, run with --gpus 1")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from dotllm_b200 import InferenceOptions, Model, StepEntry
    from dotllm_b200.config import config_from_dict
    from dotllm_b200.kernels import library, ops

    pk = peaks()
    shape_name, shape = SHAPES[args.shape]
    cfg_dict = dict(shape, num_hidden_layers=args.layers or shape["num_hidden_layers"])
    cfg = config_from_dict(cfg_dict)
    torch.cuda.set_device(0)
    t0 = time.time()
    model = Model.random(cfg, seed=0, dtype=args.dtype, device="cuda:0", on_device=True)
    esize = 2 if args.dtype == "bfloat16" else 4
    dtype_name = "bf16" if args.dtype == "bfloat16" else "fp32"
    compute_peak = pk["bf16_tflops"] if args.dtype == "bfloat16" else FP32_TFLOPS_NOMINAL
    torch.cuda.synchronize()
    print(f"[bench] model ready in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)

    steps, warmup, ctx = args.steps, args.warmup, args.context
    batches = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    reps = max(1, args.repeats)
    room = ctx + 2 * reps * steps + warmup + 128        # every timed step grows every sequence by one token
    # The cache must fit beside the weights: a batch whose sequences of `ctx` tokens would not fit
    # runs at the longest context that does (reported with its point).
    per_token = 2 * esize * cfg.num_hidden_layers * cfg.num_key_value_heads * cfg.head_dim
    free_bytes, _ = torch.cuda.mem_get_info()
    fit_tokens = int(0.85 * free_bytes) // per_token
    ctx_of = {b: min(ctx, max(256, fit_tokens // b - (room - ctx)) // 64 * 64) for b in batches}
    cache_tokens = max(b * ((ctx_of[b] + room - ctx + 63) // 64 * 64) for b in batches)
    cache = model.new_cache(max_tokens=cache_tokens, max_sequences=max(batches))
    for g in cache.kv_groups:                              # random cache contents (see the header)
        g.k.normal_(0.0, 0.5)
        g.v.normal_(0.0, 0.5)
    weight_bytes = model.decoder.weight_bytes_per_step()
    kv_bytes_per_token = cache.bytes_per_token()
    vocab = cfg.vocab_size
    gen = torch.Generator().manual_seed(1)

    # count this library's own kernel launches (the graph replays what was captured)
    launches = {"n": 0}
    real_call = library.call

    def counting_call(name, *a):
        launches["n"] += 1
        return real_call(name, *a)
    library.call = counting_call                           # every kernel module calls through library.call

    def spread(values):
        """Coefficient of variation of the repetitions (0 for a single one)."""
        return round(statistics.pstdev(values) / statistics.mean(values), 4) if len(values) > 1 else 0.0

    def decode_point(batch, measure_e2e):
        ctx = ctx_of[batch]
        seqs = [cache.open_sequence() for _ in range(batch)]
        cache.reserve([(s, ctx) for s in seqs])
        for s in seqs:
            cache.commit(s, ctx)
        tokens = torch.randint(0, vocab, (batch,), generator=gen).tolist()
        graphs = model.decode_graphs(cache)
        entries = [StepEntry(s, [t]) for s, t in zip(seqs, tokens)]
        launches["n"] = 0
        logits = graphs.run(entries)                         # captures; host tokens in
        per_replay = launches["n"] // 2                      # the eager run before capture + the capture itself
        tok_buf = graphs.token_buffer(batch)
        ops.sample(logits, out=tok_buf)
        for _ in range(warmup):
            ops.sample(graphs.run(entries, device_tokens=True), out=tok_buf)
        torch.cuda.synchronize()
        sampler = ClockSampler()
        times = []
        for _ in range(reps):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(steps):
                ops.sample(graphs.run(entries, device_tokens=True), out=tok_buf)
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop) / steps)
        clocks = sampler.stop()
        ms = min(times)
        result = {"ms": ms, "tok_s": batch * 1000.0 / ms, "clocks": clocks, "launches": steps * (per_replay + 1),
                  "mean_len": sum(s.length for s in seqs) / batch, "cv": spread(times)}
        if measure_e2e:
            host_tokens = tok_buf.tolist()
            copied = graphs.captured[batch].h2d_bytes         # counted where the copies are issued
            e2e_times = []
            for _ in range(reps):
                torch.cuda.synchronize()
                t_a = time.perf_counter()
                for _ in range(steps):
                    lg = model.step(cache, [StepEntry(s, [t]) for s, t in zip(seqs, host_tokens)], graphs=True)
                    host_tokens = ops.sample(lg).tolist()        # device -> host read of the step's result
                torch.cuda.synchronize()
                e2e_times.append((time.perf_counter() - t_a) * 1e3 / steps)
            e2e_ms = min(e2e_times)
            result["e2e"] = {"value": batch * 1000.0 / e2e_ms, "unit": "tokens/s", "ms_per_step": e2e_ms,
                             "h2d_bytes_per_step": (graphs.captured[batch].h2d_bytes - copied) // (steps * reps),
                             "d2h_bytes_per_step": 4 * batch, "cv": spread(e2e_times)}
            result["shares"] = family_shares(seqs, host_tokens)
        for s in seqs:
            cache.close_sequence(s)
        return result

    FAMILIES = (("products", ("gemm", "swiglu")), ("attention", ("attention", "rope")),
                ("norm_embed_sample", ("rmsnorm", "gather", "sample", "penalty")))

    def family_shares(seqs, host_tokens):
        """One eager decode step with a CUDA event on either side of every kernel of this library: the
        share of the summed kernel time per family.  (Eager launches do not overlap as a replayed
        graph's do, so these are shares of kernel time, not of the step's wall time.)"""
        spans = []

        def timed_call(name, *a):
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            counting_call(name, *a)
            a1.record()
            spans.append((name, a0, a1))
        library.call = timed_call
        try:
            lg = model.step(cache, [StepEntry(s, [t]) for s, t in zip(seqs, host_tokens)])
            ops.sample(lg)
            torch.cuda.synchronize()
        finally:
            library.call = counting_call
        total = sum(a0.elapsed_time(a1) for _, a0, a1 in spans) or 1.0
        shares = {}
        for family, keys in FAMILIES:
            shares[family] = round(sum(a0.elapsed_time(a1) for n, a0, a1 in spans if any(k in n for k in keys)) / total, 3)
        shares["other"] = round(max(0.0, 1.0 - sum(shares.values())), 3)
        return shares

    def prefill_flops(T, rows_out):
        """The products the step runs: Q/K/V for every token in every layer; the output projection and
        the feed-forward for every token in all layers but the last, which runs them (and the head) for
        the ``rows_out`` rows whose logits are wanted only."""
        qkv = 2 * cfg.hidden_size * (cfg.q_dim + 2 * cfg.kv_dim)
        rest = 2 * (cfg.q_dim * cfg.hidden_size + 3 * cfg.hidden_size * cfg.intermediate_size)
        L = cfg.num_hidden_layers
        return T * (L * qkv + (L - 1) * rest) + rows_out * (rest + 2 * cfg.hidden_size * vocab)

    def prefill_point(tokens=PREFILL_TOKENS):
        """One prompt of ``tokens`` tokens through model.step: best of ``reps`` after three warm-ups
        (the first is eager, the second captures the step's graph, the rest replay it)."""
        import numpy as np
        prompt = np.asarray(torch.randint(0, vocab, (tokens,), generator=gen))
        times = []
        for it in range(3 + reps):
            s = cache.open_sequence()
            torch.cuda.synchronize()
            a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            model.step(cache, [StepEntry(s, prompt)], graphs=True)       # the step's shape repeats: replayed from its graph
            b_.record()
            torch.cuda.synchronize()
            if it >= 3:
                times.append(a.elapsed_time(b_))
            cache.close_sequence(s)
        p_ms = min(times)
        T = tokens
        flops = prefill_flops(T, 1) + cfg.num_hidden_layers * 2 * T * T * cfg.q_dim
        return {"value": round(T * 1000.0 / p_ms, 1), "tokens": T, "ms": round(p_ms, 3),
                "frac": round(flops / (p_ms * 1e-3) / (compute_peak * 1e12), 4),
                "peak": pk["source"] if args.dtype == "bfloat16" else "nominal fp32", "cv": spread(times)}

    def generate_point(batch, prompt_len=128, new_tokens=256, sampled=False):
        """Tokens per second of Model.generate itself: host prompts in, host tokens out, stop tokens off.
        ``sampled``: temperature 0.8, top-k 40, top-p 0.95 and a seed instead of greedy."""
        prompts = [torch.randint(0, vocab, (prompt_len,), generator=gen).tolist() for _ in range(batch)]
        need = batch * ((prompt_len + new_tokens + 63) // 64 * 64)
        if need > cache.max_tokens:
            return None
        generator = model.generator(cache=cache, max_batch=batch)
        if sampled:
            options = InferenceOptions(temperature=0.8, top_k=40, top_p=0.95, seed=7, max_tokens=new_tokens, stop_token_ids=[])
        else:
            options = InferenceOptions(temperature=0.0, max_tokens=new_tokens, stop_token_ids=[])
        generator.generate(prompts[:batch], options)          # warm-up: captures the graph of this batch size
        times = []
        for _ in range(min(reps, 3)):
            torch.cuda.synchronize()
            t_a = time.perf_counter()
            out = generator.generate(prompts, options)
            torch.cuda.synchronize()
            times.append(time.perf_counter() - t_a)
        assert all(o.generated_token_count == new_tokens for o in out)
        t = out[0].timings
        return {"value": round(batch * new_tokens / min(times), 1), "prompt_tokens": prompt_len, "new_tokens": new_tokens,
                "decode_tok_s": round(batch * t.decode_steps / (t.decode_ms / 1e3), 1), "prefill_ms": round(t.prefill_ms, 2),
                "sampling_ms": round(t.sampling_ms, 2), "cv": spread(times)}

    if args.workload == "short-prompts":
        return short_prompt_workload(args, model, cfg, gen, shape_name, dtype_name)
    if args.workload == "staggered":
        return staggered_workload(args, model, cfg, gen, shape_name, dtype_name)
    if args.workload == "unequal":
        return unequal_workload(args, model, cache, cfg, gen, pk, shape_name, dtype_name, compute_peak, weight_bytes, prefill_flops)

    if args.only_prefill:
        print(json.dumps({"prefill": prefill_point(args.prefill_tokens), "layers": cfg.num_hidden_layers}))
        return 0

    main_point = decode_point(args.batch, True)
    points = {}
    prefill = None
    generate = {}
    if not args.no_points:
        for b in batches:
            if b != args.batch:
                name = f"decode_b{b}" if ctx_of[b] == ctx else f"decode_b{b}_ctx{ctx_of[b]}"
                points[name] = round(decode_point(b, False)["tok_s"], 1)
        points[f"decode_b{args.batch}"] = round(main_point["tok_s"], 1)
        prefill = prefill_point()
        if not args.no_generate:
            for b in sorted({args.batch, 64}):
                g = generate_point(b)
                if g is not None:
                    generate[f"b{b}"] = g
            g = generate_point(64, sampled=True)
            if g is not None:
                generate["b64_sampled"] = g

    step_bytes = weight_bytes + args.batch * main_point["mean_len"] * kv_bytes_per_token
    achieved = step_bytes / (main_point["ms"] * 1e-3) / 1e9
    line = {
        "metric": "decode tokens/s", "value": round(main_point["tok_s"], 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(main_point["ms"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_name,
        "data": "synthetic: seeded random weights, random token ids, random cache contents",
        "config": {"model": shape_name, "layers": cfg.num_hidden_layers,
                   "layers_full": shape["num_hidden_layers"], "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": vocab,
                   "global_batch": args.batch, "seq_len": ctx_of[args.batch], "parallelism": "none (1 GPU)",
                   "weights": dtype_name, "cache": f"{dtype_name} pages of 64 tokens",
                   "l2": "inputs larger than L2 (all weights are read every step)",
                   "decode": "CUDA graph replay, one captured graph per batch size",
                   "prefill_tokens": PREFILL_TOKENS},
        "repeats": reps, "cv": main_point["cv"],
        "clocks": main_point["clocks"],
        "e2e": main_point.get("e2e"),
        "gpu_launches": main_point["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"],
                     "bytes_per_step": int(step_bytes)},
        "shares": main_point.get("shares"),
    }
    if prefill is not None:
        line["prefill"] = prefill
        line["points"] = points
    if generate:
        line["generate"] = generate
    print(json.dumps(line))
    return 0


def short_prompt_workload(args, model, cfg, gen, shape_name, dtype_name):
    """The time from a prompt's tokens on the host to its first token on the host, for single prompts
    of random lengths in five ranges: stepped eagerly (the host launches every kernel) and through
    captured steps that prompts of other lengths share (`Model.step(graphs=True)`: a prompt's tokens
    are filled up to the next multiple of 64, a power of two below, and forgotten after the step).
    Median of ten prompts after four that warm up and capture.  Prints its own JSON line."""
    import random
    import torch
    from dotllm_b200 import StepEntry
    rng = random.Random(3)
    out = {}
    for lo, hi in ((20, 32), (65, 128), (193, 256), (449, 512), (961, 1024)):
        cell = {}
        for label, graphs in (("eager_ms", False), ("captured_ms", True)):
            cache = model.new_cache(max_tokens=4096)
            times = []
            for _ in range(14):
                prompt = torch.randint(0, cfg.vocab_size, (rng.randint(lo, hi),), generator=gen).tolist()
                seq = cache.open_sequence()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                first = int(model.step(cache, [StepEntry(seq, prompt)], graphs=graphs).argmax())
                times.append((time.perf_counter() - t0) * 1e3)
                cache.close_sequence(seq)
            assert 0 <= first < cfg.vocab_size
            cell[label] = round(sorted(times[4:])[5], 3)
            del cache
        out[f"{lo}-{hi}"] = cell
    print(json.dumps({"metric": "time to the first token of one short prompt", "model": shape_name, "dtype": dtype_name, "unit": "ms",
                      "prompt_tokens": out, "data": "synthetic: seeded random weights, prompt lengths and token ids"}))
    return 0


def staggered_workload(args, model, cfg, gen, shape_name, dtype_name):
    """`Model.generate` on 64 prompts of 128 tokens whose requests end one by one, five steps apart
    (request i generates 40 + 5 i tokens: 12,640 in all, 355 steps, every batch size from 64 to 1):
    what the loop's ways of stepping cost and give when the batch keeps shrinking.  Three generators,
    each on a cache of its own, each called four times: without graphs; with graphs of a few widths;
    with those and every step started before the host has the tokens of the step before it.  The
    first call of a generator captures its graphs.  Prints its own JSON line."""
    import torch
    from dotllm_b200 import InferenceOptions
    n = 64
    prompts = [torch.randint(0, cfg.vocab_size, (128,), generator=gen).tolist() for _ in range(n)]
    options = [InferenceOptions(temperature=0.0, max_tokens=40 + 5 * i, stop_token_ids=[]) for i in range(n)]
    total = sum(o.max_tokens for o in options)
    out = {}
    for label, use_graphs, ahead in (("eager", False, False), ("graphs", True, False), ("graphs_ahead", True, True)):
        cache = model.new_cache(max_tokens=n * 512, max_sequences=n)
        generator = model.generator(cache=cache, max_batch=n, use_graphs=use_graphs, ahead=ahead)
        seconds = []
        for _ in range(4):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            results = generator.generate(prompts, options)
            torch.cuda.synchronize()
            seconds.append(time.perf_counter() - t0)
            assert sum(r.generated_token_count for r in results) == total
        runner = getattr(cache, "_decode_graphs", None)
        out[label] = {"first_call": round(total / seconds[0], 1), "later_calls": round(total / min(seconds[1:]), 1),
                      "first_call_s": round(seconds[0], 3), "later_call_s": round(min(seconds[1:]), 3),
                      "graphs": len(runner.captured) if runner is not None else 0, "steps_ahead": generator.ahead_steps}
        del generator, cache
    print(json.dumps({"metric": "generate tokens/s while 64 requests end one by one", "model": shape_name, "dtype": dtype_name,
                      "requests": n, "prompt_tokens": 128, "new_tokens": total, "unit": "tokens/s", **out,
                      "data": "synthetic: seeded random weights and token ids; greedy, stop tokens off"}))
    return 0


def unequal_workload(args, model, cache, cfg, gen, pk, shape_name, dtype_name, compute_peak, weight_bytes, prefill_flops):
    """64 prompts with lengths uniform in [16, 2048] in ONE prefill step, then 256 decode steps at batch
    64 (the Llama-3.2-1B-shaped workload).  Prints its own JSON line."""
    import numpy as np
    import torch
    from dotllm_b200 import StepEntry
    from dotllm_b200.kernels import ops
    n_seqs, n_decode = 64, 256
    lens = torch.randint(16, 2049, (n_seqs,), generator=gen).tolist()
    prompts = [np.asarray(torch.randint(0, cfg.vocab_size, (n,), generator=gen)) for n in lens]
    need = sum((n + n_decode + 63) // 64 * 64 for n in lens)
    big = model.new_cache(max_tokens=need, max_sequences=n_seqs) if need > cache.max_tokens else cache
    results = {"prefill_ms": [], "decode_ms": [], "plan_ms": []}
    from dotllm_b200.engine.step import plan_step
    for rep in range(1 + min(args.repeats, 3)):
        seqs = [big.open_sequence() for _ in prompts]
        entries = [StepEntry(s, p) for s, p in zip(seqs, prompts)]
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_host = time.perf_counter()
        a.record()
        logits = model.step(big, entries)
        b.record()
        torch.cuda.synchronize()
        graphs = model.decode_graphs(big)
        tokens = ops.sample(logits).tolist()
        dec = [StepEntry(s, [t]) for s, t in zip(seqs, tokens)]
        lg = graphs.run(dec)
        tok_buf = graphs.token_buffer(n_seqs)
        ops.sample(lg, out=tok_buf)
        torch.cuda.synchronize()
        c, d = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c.record()
        for _ in range(n_decode - 1):
            ops.sample(graphs.run(dec, device_tokens=True), out=tok_buf)
        d.record()
        torch.cuda.synchronize()
        mean_len = sum(s.length for s in seqs) / n_seqs - n_decode / 2
        for s in seqs:
            big.close_sequence(s)
        # what planning alone costs on the host, without the model
        seqs = [big.open_sequence() for _ in prompts]
        t0 = time.perf_counter()
        plan_step([StepEntry(s, p) for s, p in zip(seqs, prompts)], big, cfg.vocab_size, 1 << 30, model.runtime.device)
        plan_ms = (time.perf_counter() - t0) * 1e3
        for s in seqs:
            big.close_sequence(s)
        if rep:                                              # the first round warms up (captures the graph)
            results["prefill_ms"].append(a.elapsed_time(b))
            results["decode_ms"].append(c.elapsed_time(d) / (n_decode - 1))
            results["plan_ms"].append(plan_ms)
    total = sum(lens)
    p_ms, d_ms = min(results["prefill_ms"]), min(results["decode_ms"])
    flops = prefill_flops(total, n_seqs) + cfg.num_hidden_layers * sum(2 * n * n * cfg.q_dim for n in lens)
    step_bytes = weight_bytes + n_seqs * mean_len * big.bytes_per_token()
    print(json.dumps({
        "metric": "unequal batch: prefill tokens/s and decode tokens/s", "model": shape_name, "dtype": dtype_name,
        "sequences": n_seqs, "prompt_tokens": total, "decode_steps": n_decode,
        "prefill": {"value": round(total * 1e3 / p_ms, 1), "ms": round(p_ms, 2), "planning_ms": round(min(results["plan_ms"]), 2),
                    "frac": round(flops / (p_ms * 1e-3) / (compute_peak * 1e12), 4)},
        "decode": {"value": round(n_seqs * 1e3 / d_ms, 1), "ms_per_step": round(d_ms, 4),
                   "roofline_frac": round(step_bytes / (d_ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)},
        "data": "synthetic: seeded random weights, seeded prompt lengths and token ids"}))
    return 0


def cpp_model_tokens_per_second(tmp, folder, cfg, tokens):
    """The one-file C++ float32 model under tests/cpu_reference, compiled here and timed on one prompt."""
    import shutil
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        return None
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from test_cpu_reference import SOURCE, arguments
    exe = tmp / "llama_f32"
    if subprocess.run([cxx, "-O2", "-std=c++17", "-o", str(exe), str(SOURCE)], capture_output=True).returncode != 0:
        return None
    (tmp / "tokens.txt").write_text(" ".join(str(t) for t in tokens))
    res = subprocess.run([str(exe), str(folder / "model.safetensors"), str(tmp / "tokens.txt"), str(tmp / "out.f32"), *arguments(cfg)],
                         capture_output=True, text=True)
    return json.loads(res.stdout)["tokens_per_second"] if res.returncode == 0 else None


def plain_cpu_baseline():
    """The plain implementation (tests/plain_llama.py, float32, PyTorch on the host's cores) timed on the
    tiny test models and on a short prompt through one Llama-3.2-1B-shaped layer stack: the CPU line
    that stands where the reference's own CPU numbers would."""
    import tempfile
    from pathlib import Path
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_llama
    import tiny_models
    from dotllm_b200.config import config_from_dict
    from dotllm_b200.weights import write_random_model
    out = {"impl": "plain-cpu", "threads": torch.get_num_threads(), "cells": {}}
    with tempfile.TemporaryDirectory() as tmp:
        for which, lens, n_new in (("A", tiny_models.TINY_A_PROMPTS, tiny_models.TINY_A_DECODE),
                                   ("B", tiny_models.TINY_B_PROMPTS, tiny_models.TINY_B_DECODE)):
            folder = tiny_models.make_folder(Path(tmp), which, seed=0)
            cfg, weights = plain_llama.read_model_folder(folder)
            prompts = [tiny_models.random_tokens(n, cfg["vocab_size"], 3 + n) for n in lens]
            t0 = time.perf_counter()
            for p in prompts:
                plain_llama.forward(cfg, weights, p)
            prefill_s = time.perf_counter() - t0
            t0 = time.perf_counter()
            for p in prompts:
                plain_llama.greedy_generate(cfg, weights, p, n_new)
            out["cells"][f"tiny_{which}"] = {"prefill_tok_s": round(sum(lens) / prefill_s, 1),
                                             "generate_tok_s_no_cache": round(len(lens) * n_new / (time.perf_counter() - t0), 1)}
            cpp = cpp_model_tokens_per_second(Path(tmp), folder, cfg, prompts[-1])
            if cpp is not None:
                out["cells"][f"tiny_{which}"]["cpp_f32_prefill_tok_s"] = cpp
        one_b = dict(LLAMA_32_1B, num_hidden_layers=2, max_position_embeddings=4096)
        folder = write_random_model(Path(tmp) / "1b", config_from_dict(one_b), seed=0, dtype=torch.bfloat16)
        cfg, weights = plain_llama.read_model_folder(folder)
        prompt = tiny_models.random_tokens(128, cfg["vocab_size"], 9)
        plain_llama.forward(cfg, weights, prompt[:8])
        t0 = time.perf_counter()
        plain_llama.forward(cfg, weights, prompt)
        dt = time.perf_counter() - t0
        out["cells"]["llama_3.2_1b_shape_2_of_16_layers"] = {"prefill_tokens": 128, "seconds": round(dt, 3),
                                                             "prefill_tok_s_2_layers_and_head": round(128 / dt, 1)}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
