"""Command line in the manner of ``dotllm run`` (src/DotLLM.Cli/Commands/RunCommand.cs:26-171):

    python -m dotllm_b200 run <model_dir> --prompt-ids 1,2,3 -n 64 -t 0.8 --top-k 40 -s 7 --json
    python -m dotllm_b200 random <config.json> <out_dir> --seed 0 --dtype bfloat16

The option names, defaults and meanings of ``run`` are the reference's where it has them
(--max-tokens/-n 128, --temp/-t 0 = greedy, --top-k 0, --top-p 1.0, --min-p 0, --repeat-penalty 1.0,
--repeat-last-n 0, --seed/-s, --device/-d, --json).  The reference takes text and a tokenizer; this
library works on token ids, given like the reference's debug command takes them
(src/DotLLM.Cli/Commands/Debug/DebugForwardPassCommand.cs:93-99).  The default device is the GPU:
there is no CPU backend here.
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def _parse_ids(text):
    text = text.strip().lstrip("[").rstrip("]")
    return [int(t) for t in text.replace(",", " ").split()] if text else []


def _read_prompts(args):
    prompts = []
    for p in args.prompt_ids or []:
        prompts.append(_parse_ids(p))
    if args.prompt_file:
        data = json.loads(open(args.prompt_file).read())
        if data and isinstance(data[0], int):
            data = [data]
        prompts.extend([int(t) for t in p] for p in data)
    if not prompts:
        raise SystemExit("error: give --prompt-ids (repeatable) or --prompt-file")
    return prompts


def run_command(args):
    from . import InferenceOptions, Model
    t0 = time.perf_counter()
    model = Model.load(args.model, dtype=args.dtype, device=args.device)
    load_ms = (time.perf_counter() - t0) * 1e3
    prompts = _read_prompts(args)
    options = InferenceOptions(temperature=args.temp, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p,
                               repetition_penalty=args.repeat_penalty,
                               repetition_penalty_window=args.repeat_last_n, max_tokens=args.max_tokens,
                               seed=args.seed,
                               stop_token_ids=None if args.stop_ids is None else _parse_ids(args.stop_ids))
    longest = max(len(p) for p in prompts) + args.max_tokens
    per_request = (min(longest, model.spec.max_positions) + 63) // 64 * 64
    batch = min(len(prompts), args.max_batch)
    cache = model.new_cache(max_tokens=args.cache_tokens or per_request * batch)
    generator = model.generator(cache=cache, max_batch=args.max_batch)
    stream = (lambda i, tok: print(f"[{i}] {tok}", flush=True)) if args.stream and not args.json else None
    t0 = time.perf_counter()
    responses = generator.generate(prompts, options, on_token=stream)
    total_ms = (time.perf_counter() - t0) * 1e3
    results = []
    for p, r in zip(prompts, responses):
        t = r.timings
        results.append({
            "prompt_token_ids": p, "generated_token_ids": r.generated_token_ids,
            "finish_reason": r.finish_reason.value,
            "usage": {"prompt_tokens": r.prompt_token_count, "completion_tokens": r.generated_token_count,
                      "total_tokens": r.prompt_token_count + r.generated_token_count},
            "timings": {"load_ms": load_ms, "prefill_ms": t.prefill_ms, "decode_ms": t.decode_ms,
                        "sampling_ms": t.sampling_ms, "total_ms": total_ms,
                        "prefill_tok_s": t.prefill_tokens_per_sec, "decode_tok_s": t.decode_tokens_per_sec,
                        "batch_size": t.batch_size}})
    if args.json:                                           # RunJsonResult.cs:9-60
        doc = {"model": args.model, "dtype": args.dtype, "results": results,
               "memory": {"weights_bytes": model.decoder.weight_bytes_per_step(), "kv_cache_bytes": cache.bytes()}}
        print(json.dumps(doc))
    else:
        for i, r in enumerate(results):
            print(f"--- request {i}: {r['usage']['prompt_tokens']} prompt tokens, "
                  f"{r['usage']['completion_tokens']} generated, finish: {r['finish_reason']}")
            print(" ".join(str(t) for t in r["generated_token_ids"]))
        t = results[0]["timings"]
        print(f"load {load_ms:.0f} ms | prefill {t['prefill_ms']:.1f} ms ({t['prefill_tok_s']:.0f} tok/s) | "
              f"decode {t['decode_ms']:.1f} ms ({t['decode_tok_s']:.1f} tok/s per sequence, "
              f"batch {t['batch_size']}) | sampling {t['sampling_ms']:.1f} ms", file=sys.stderr)
    return 0


def random_command(args):
    import torch
    from .config import config_from_dict
    from .weights import write_random_model
    cfg = config_from_dict(json.loads(open(args.config).read()))
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    folder = write_random_model(args.out, cfg, args.seed, dtype=dtype)
    print(folder)
    return 0


def build_parser():
    parser = argparse.ArgumentParser(prog="dotllm_b200")
    sub = parser.add_subparsers(dest="command", required=True)
    run = sub.add_parser("run", help="generate from token-id prompts")
    run.add_argument("model", help="folder with config.json and model.safetensors")
    run.add_argument("--prompt-ids", "-p", action="append", help='token ids, e.g. "1,2,3" (repeat for a batch)')
    run.add_argument("--prompt-file", help="JSON file: a list of token ids, or a list of such lists")
    run.add_argument("--max-tokens", "-n", type=int, default=128, help="maximum number of tokens to generate")
    run.add_argument("--temp", "-t", type=float, default=0.0, help="sampling temperature; 0 = greedy")
    run.add_argument("--top-k", type=int, default=0, help="top-K sampling; 0 = disabled")
    run.add_argument("--top-p", type=float, default=1.0, help="top-P (nucleus) threshold")
    run.add_argument("--min-p", type=float, default=0.0, help="min-P threshold; 0 = disabled")
    run.add_argument("--repeat-penalty", type=float, default=1.0, help="repetition penalty; 1.0 = disabled")
    run.add_argument("--repeat-last-n", type=int, default=0, help="penalty lookback; 0 = full history")
    run.add_argument("--seed", "-s", type=int, default=None, help="seed for reproducible sampling")
    run.add_argument("--device", "-d", default="gpu", help="'gpu', 'gpu:0', 'cuda:1' ...")
    run.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    run.add_argument("--stop-ids", default=None, help='stop token ids, e.g. "2,128009"; default: the model\'s eos ids')
    run.add_argument("--max-batch", type=int, default=64, help="most sequences in one batch")
    run.add_argument("--cache-tokens", type=int, default=0, help="cache size in tokens; 0 = what the prompts need")
    run.add_argument("--stream", action="store_true", help="print tokens as they are generated")
    run.add_argument("--json", action="store_true", help="print one JSON object and nothing else")
    run.set_defaults(func=run_command)
    rnd = sub.add_parser("random", help="write a model folder with random weights")
    rnd.add_argument("config", help="a config.json")
    rnd.add_argument("out", help="folder to write")
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    rnd.set_defaults(func=random_command)
    return parser


def main(argv=None):
    args = build_parser().parse_args(argv)
    return args.func(args)


if __name__ == "__main__":
    sys.exit(main())
