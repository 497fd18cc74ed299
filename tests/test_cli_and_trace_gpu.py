"""bin/trace_run and the command line, run as a user runs them (separate processes)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama
import tiny_models
from engine_checks import TOL, greedy_ok

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def replay(folder, dtype, steps, out_dir, max_tokens):
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(folder), "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", str(max_tokens)],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    return proc


def read(out_dir, step, vocab):
    return torch.from_numpy(np.fromfile(out_dir / f"{step}.f32", dtype="<f4").reshape(-1, vocab).copy())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B", "D"])
def test_trace_run_whole_tail_and_batches(tmp_path, which, dtype):
    tdtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    folder = tiny_models.make_folder(tmp_path, which, seed=4, dtype=tdtype)
    cfg, weights = plain_llama.read_model_folder(folder)
    vocab = cfg["vocab_size"]
    lens = [40, 7, 100, 65, 33, 90]
    reqs = {f"r{i}": tiny_models.random_tokens(n, vocab, 200 + i) for i, n in enumerate(lens)}
    refs = {k: plain_llama.forward(cfg, weights, v) for k, v in reqs.items()}
    tol = TOL[tdtype]

    # whole: each request alone, every position wanted
    steps = [{"step": i, "entries": [{"id": k, "tokens": v, "want": list(range(len(v)))}], "end": [k]}
             for i, (k, v) in enumerate(reqs.items())]
    out = tmp_path / f"whole_{which}_{dtype}"
    replay(folder, dtype, steps, out, 128)
    for i, k in enumerate(reqs):
        assert float((read(out, i, vocab) - refs[k]).abs().max()) <= tol, ("whole", k)

    # the last 32 tokens one by one
    steps, expect, n = [], [], 0
    for k, v in reqs.items():
        head = max(0, len(v) - 32)
        if head:
            steps.append({"step": n, "entries": [{"id": k, "tokens": v[:head], "want": [head - 1]}], "end": []})
            expect.append((n, k, [head - 1]))
            n += 1
        for t in range(head, len(v)):
            steps.append({"step": n, "entries": [{"id": k, "tokens": [v[t]], "want": [0]}],
                          "end": [k] if t == len(v) - 1 else []})
            expect.append((n, k, [t]))
            n += 1
    out = tmp_path / f"tail_{which}_{dtype}"
    replay(folder, dtype, steps, out, 128)
    for step, k, rows in expect:
        assert float((read(out, step, vocab) - refs[k][rows]).abs().max()) <= tol, ("tail", k, rows)

    # batches of unequal lengths, shorter requests end earlier, one batch after another in a
    # cache that holds one batch only
    steps, expect, n = [], [], 0
    names = list(reqs)
    for batch in (names[:3], names[3:]):
        tails = {k: min(len(reqs[k]) - 1, 4 + 9 * j) for j, k in enumerate(batch)}
        heads = {k: len(reqs[k]) - tails[k] for k in batch}
        steps.append({"step": n, "entries": [{"id": k, "tokens": reqs[k][:heads[k]], "want": [0, heads[k] - 1]}
                                             for k in batch], "end": [k for k in batch if tails[k] == 0]})
        expect.append((n, [(k, r) for k in batch for r in (0, heads[k] - 1)]))
        n += 1
        done = {k: 0 for k in batch}
        live = [k for k in batch if tails[k] > 0]
        while live:
            entries = [{"id": k, "tokens": [reqs[k][heads[k] + done[k]]], "want": [0]} for k in live]
            expect.append((n, [(k, heads[k] + done[k]) for k in live]))
            for k in live:
                done[k] += 1
            ending = [k for k in live if done[k] == tails[k]]
            steps.append({"step": n, "entries": entries, "end": ending})
            live = [k for k in live if k not in ending]
            n += 1
    need = max(sum((len(reqs[k]) + 63) // 64 * 64 for k in b) for b in (names[:3], names[3:]))
    out = tmp_path / f"batch_{which}_{dtype}"
    replay(folder, dtype, steps, out, need)
    for step, rows in expect:
        got = read(out, step, vocab)
        want = torch.stack([refs[k][r] for k, r in rows])
        assert float((got - want).abs().max()) <= tol, ("batched", step, rows)


def test_trace_run_fails_loudly(tmp_path):
    folder = tiny_models.make_folder(tmp_path, "A", seed=4)
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(folder), "--dtype", "float32",
                           "--out", str(tmp_path / "o"), "--max-tokens", "64"],
                          input=json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [999], "want": [0]}], "end": []}) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode != 0 and "vocabulary" in proc.stderr and "done" not in proc.stdout


def test_run_command_json(tmp_path):
    folder = tiny_models.make_folder(tmp_path, "B", seed=5, dtype=torch.bfloat16)
    cfg, weights = plain_llama.read_model_folder(folder)
    p1, p2 = tiny_models.random_tokens(12, 384, 1), tiny_models.random_tokens(3, 384, 2)
    proc = subprocess.run([sys.executable, "-m", "dotllm_b200", "run", str(folder), "-p", ",".join(map(str, p1)),
                           "-p", " ".join(map(str, p2)), "-n", "5", "-t", "0", "--stop-ids", "", "--json"],
                          cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    doc = json.loads(proc.stdout)
    assert len(doc["results"]) == 2
    for prompt, r in zip((p1, p2), doc["results"]):
        assert r["usage"] == {"prompt_tokens": len(prompt), "completion_tokens": 5, "total_tokens": len(prompt) + 5}
        assert r["finish_reason"] == "length" and r["timings"]["decode_tok_s"] > 0
        ref = plain_llama.forward(cfg, weights, prompt + r["generated_token_ids"])
        for i, tok in enumerate(r["generated_token_ids"]):
            row = ref[len(prompt) - 1 + i]
            assert greedy_ok(row, tok, torch.bfloat16), (i, tok, int(row.argmax()))
    sampled = subprocess.run([sys.executable, "-m", "dotllm_b200", "run", str(folder), "-p", "1,2,3", "-n", "8",
                              "-t", "0.8", "--top-k", "20", "--top-p", "0.9", "--min-p", "0.02",
                              "--repeat-penalty", "1.1", "--repeat-last-n", "4", "-s", "7", "--json"],
                             cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert sampled.returncode == 0, sampled.stderr[-2000:]
    again = subprocess.run([sys.executable, "-m", "dotllm_b200", "run", str(folder), "-p", "1,2,3", "-n", "8",
                            "-t", "0.8", "--top-k", "20", "--top-p", "0.9", "--min-p", "0.02",
                            "--repeat-penalty", "1.1", "--repeat-last-n", "4", "-s", "7", "--json"],
                           cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert json.loads(sampled.stdout)["results"][0]["generated_token_ids"] == \
        json.loads(again.stdout)["results"][0]["generated_token_ids"]
