"""The one-file C++ float32 model (tests/cpu_reference/llama_f32.cpp) against the plain implementation
in Python: two statements of the reference's formulas that share nothing, on both tiny models."""
import json
import shutil
import subprocess

import numpy as np
import pytest
import torch

import plain_llama
import tiny_models
from pathlib import Path

SOURCE = Path(__file__).parent / "cpu_reference" / "llama_f32.cpp"


def build(tmp_path):
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        pytest.skip("no C++ compiler")
    exe = tmp_path / "llama_f32"
    res = subprocess.run([cxx, "-O2", "-std=c++17", "-o", str(exe), str(SOURCE)], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return exe


def arguments(cfg):
    args = {"layers": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg.get("num_key_value_heads") or cfg["num_attention_heads"],
            "head_dim": cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "eps": cfg.get("rms_norm_eps", 1e-5),
            "theta": cfg.get("rope_theta", 10000.0), "tied": int(bool(cfg.get("tie_word_embeddings", False))), "scaling": 0}
    s = cfg.get("rope_scaling")
    if s:
        args.update(scaling=1, factor=s["factor"], low=s["low_freq_factor"], high=s["high_freq_factor"],
                    original=s["original_max_position_embeddings"])
    return [f"{k}={v!r}" for k, v in args.items()]


@pytest.mark.parametrize("which,n_tokens", [("A", 40), ("B", 100)])
def test_cpp_model_agrees_with_the_plain_implementation(tmp_path, which, n_tokens):
    exe = build(tmp_path)
    folder = tiny_models.make_folder(tmp_path, which, seed=6, dtype=torch.float32)
    cfg, weights = plain_llama.read_model_folder(folder)
    tokens = tiny_models.random_tokens(n_tokens, cfg["vocab_size"], seed=60)      # B: past the scaling's original length
    (tmp_path / "tokens.txt").write_text(" ".join(str(t) for t in tokens))
    res = subprocess.run([str(exe), str(folder / "model.safetensors"), str(tmp_path / "tokens.txt"), str(tmp_path / "out.f32"),
                          *arguments(cfg)], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    assert json.loads(res.stdout)["tokens"] == n_tokens
    got = torch.from_numpy(np.fromfile(tmp_path / "out.f32", dtype="<f4").reshape(n_tokens, cfg["vocab_size"]))
    want = plain_llama.forward(cfg, weights, tokens)
    err = float((got - want).abs().max())
    assert err <= 5e-6, f"the C++ model and the plain implementation differ by {err:.3e}"
    # a tensor the program needs and does not find is a loud failure
    bad = subprocess.run([str(exe), str(folder / "model.safetensors"), str(tmp_path / "tokens.txt"), str(tmp_path / "out.f32"),
                          *[a if not a.startswith("layers=") else "layers=9" for a in arguments(cfg)]], capture_output=True, text=True)
    assert bad.returncode != 0 and "missing tensor" in bad.stderr
