"""Decode and prefill throughput of the Llama-3.1-8B-shaped model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 8192] [--layers L]

A "step" is one decode step: one new token for each of ``batch`` sequences that already hold
``context`` tokens.  ``value`` is decoded tokens per second, timed on the device with CUDA events
over K consecutive steps (every step reads all weights, far more than the L2 holds).  ``e2e`` is
the same through the public entry point with host token ids in and out every step.  The line also
carries a 2,048-token prefill, decode at batch 1 and 64, and the decode step's HBM roofline.

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
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes: the 8B default, or 1b / 13b")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (0: all of them)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points and the prefill")
    ap.add_argument("--only-prefill", action="store_true", help="run only the 2,048-token prefill (for profiling)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference",
                          "unavailable": "kkokosa/dotLLM is a .NET 10 program reading GGUF checkpoints; no .NET SDK, "
                                         "no checkpoint and no network exist here, so it cannot be installed or run"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU library: --gpus {args.gpus} is not supported, run with --gpus 1")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from dotllm_b200 import Model, StepEntry
    from dotllm_b200.config import config_from_dict
    from dotllm_b200.kernels import library, ops

    pk = peaks()
    shape_name, shape = SHAPES[args.shape]
    cfg_dict = dict(shape, num_hidden_layers=args.layers or shape["num_hidden_layers"])
    cfg = config_from_dict(cfg_dict)
    torch.cuda.set_device(0)
    t0 = time.time()
    model = Model.random(cfg, seed=0, dtype="bfloat16", device="cuda:0", on_device=True)
    torch.cuda.synchronize()
    print(f"[bench] model ready in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)

    steps, warmup, ctx = args.steps, args.warmup, args.context
    batches = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    room = ctx + 4 * (steps + warmup) + 128
    # The cache must fit beside the weights: a batch whose sequences of `ctx` tokens would not fit
    # runs at the longest context that does (reported with its point).
    per_token = 2 * 2 * cfg.num_hidden_layers * cfg.num_key_value_heads * cfg.head_dim
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
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            ops.sample(graphs.run(entries, device_tokens=True), out=tok_buf)
        stop.record()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        ms = start.elapsed_time(stop) / steps
        result = {"ms": ms, "tok_s": batch * 1000.0 / ms, "clocks": clocks, "launches": steps * (per_replay + 1),
                  "mean_len": sum(s.length for s in seqs) / batch}
        if measure_e2e:
            host_tokens = tok_buf.tolist()
            copied = graphs.captured[batch].h2d_bytes         # counted where the copies are issued
            torch.cuda.synchronize()
            t_a = time.perf_counter()
            for _ in range(steps):
                lg = model.step(cache, [StepEntry(s, [t]) for s, t in zip(seqs, host_tokens)], graphs=True)
                host_tokens = ops.sample(lg).tolist()        # device -> host read of the step's result
            torch.cuda.synchronize()
            e2e_ms = (time.perf_counter() - t_a) * 1e3 / steps
            result["e2e"] = {"value": batch * 1000.0 / e2e_ms, "unit": "tokens/s", "ms_per_step": e2e_ms,
                             "h2d_bytes_per_step": (graphs.captured[batch].h2d_bytes - copied) // steps,
                             "d2h_bytes_per_step": 4 * batch}
        for s in seqs:
            cache.close_sequence(s)
        return result

    def prefill_point():
        """One prompt of PREFILL_TOKENS tokens through model.step: best of three after three warm-ups."""
        prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
        times = []
        for it in range(3 + 3):
            s = cache.open_sequence()
            torch.cuda.synchronize()
            a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            model.step(cache, [StepEntry(s, prompt)])
            b_.record()
            torch.cuda.synchronize()
            if it >= 3:
                times.append(a.elapsed_time(b_))
            cache.close_sequence(s)
        p_ms = min(times)
        T = PREFILL_TOKENS
        per_layer = 2 * T * (cfg.hidden_size * (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim * cfg.hidden_size
                             + 3 * cfg.hidden_size * cfg.intermediate_size) + 2 * T * T * cfg.q_dim
        flops = cfg.num_hidden_layers * per_layer + 2 * cfg.hidden_size * vocab
        return {"value": round(T * 1000.0 / p_ms, 1), "tokens": T, "ms": round(p_ms, 3),
                "frac": round(flops / (p_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "peak": pk["source"]}

    if args.only_prefill:
        print(json.dumps({"prefill": prefill_point(), "layers": cfg.num_hidden_layers}))
        return 0

    main_point = decode_point(args.batch, True)
    points = {}
    prefill = None
    if not args.no_points:
        for b in batches:
            if b != args.batch:
                name = f"decode_b{b}" if ctx_of[b] == ctx else f"decode_b{b}_ctx{ctx_of[b]}"
                points[name] = round(decode_point(b, False)["tok_s"], 1)
        points[f"decode_b{args.batch}"] = round(main_point["tok_s"], 1)
        prefill = prefill_point()

    step_bytes = weight_bytes + args.batch * main_point["mean_len"] * kv_bytes_per_token
    achieved = step_bytes / (main_point["ms"] * 1e-3) / 1e9
    line = {
        "metric": "decode tokens/s", "value": round(main_point["tok_s"], 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(main_point["ms"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights, random token ids, random cache contents",
        "config": {"model": shape_name, "layers": cfg.num_hidden_layers,
                   "layers_full": shape["num_hidden_layers"], "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": vocab,
                   "global_batch": args.batch, "seq_len": ctx_of[args.batch], "parallelism": "none (1 GPU)",
                   "weights": "bf16", "cache": "bf16 pages of 64 tokens",
                   "l2": "inputs larger than L2 (all weights are read every step)",
                   "decode": "CUDA graph replay, one captured graph per batch size",
                   "prefill_tokens": PREFILL_TOKENS},
        "clocks": main_point["clocks"],
        "e2e": main_point.get("e2e"),
        "gpu_launches": main_point["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"],
                     "bytes_per_step": int(step_bytes)},
    }
    if prefill is not None:
        line["prefill"] = prefill
        line["points"] = points
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
