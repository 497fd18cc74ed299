"""Plain, slow Llama dense decoder: whole sequences, no cache, one function per part.

This is the oracle that the engine is compared with.  It shares no code with
the package: it reads ``config.json`` as a plain dict, reads the safetensors
file with its own few lines, and computes every part with elementary torch
operations on the CPU in float32 (tables in float64).

It rests on the formulas of kkokosa/dotLLM's scalar reference kernels; the
reference's model code is C#/.NET and cannot be compiled or imported here.
What can be compiled are its FP32 CUDA kernels for every part that is not a
matrix product: tests/golden/reference_kernels.py runs them unmodified, their
outputs are committed beside it, and tests/test_plain_llama.py holds the
functions below to those outputs (norm, rotation, attention, gating, add,
lookup).  Every function names the reference lines that it restates.  The reference applies no RoPE frequency
rescaling (src/DotLLM.Cpu/Kernels/RoPE.md:303); the ``llama3`` rescaling below
follows the rule published with the Llama 3.1 checkpoints' ``rope_scaling``
block and has no reference counterpart.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


# --------------------------------------------------------------------------- io
_ST_DTYPES = {"F32": (np.float32, 4), "BF16": (np.uint16, 2), "F16": (np.float16, 2),
              "I32": (np.int32, 4), "I64": (np.int64, 8)}


def read_model_folder(folder):
    """config.json as a dict and every tensor of model.safetensors widened to float32."""
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    (header_len,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + header_len])
    base = 8 + header_len
    weights = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        np_dtype, _ = _ST_DTYPES[meta["dtype"]]
        lo, hi = meta["data_offsets"]
        arr = np.frombuffer(raw[base + lo:base + hi], dtype=np_dtype).reshape(meta["shape"])
        if meta["dtype"] == "BF16":
            arr = (arr.astype(np.uint32) << 16).view(np.float32)
        weights[name] = torch.from_numpy(np.array(arr, dtype=np.float32))
    return config, weights


# ------------------------------------------------------------------ the parts
def embed(table, tokens):
    """h[t,:] = E[token[t],:], no scale (src/DotLLM.Models/Architectures/TransformerModel.cs:729-749)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    if tokens.numel() and (int(tokens.min()) < 0 or int(tokens.max()) >= table.shape[0]):
        raise IndexError("token id outside the vocabulary")
    return table[tokens].clone()


def rms_norm(x, gain, eps):
    """y_i = x_i / sqrt(mean(x^2) + eps) * w_i, eps inside the root
    (src/DotLLM.Cpu/Kernels/RmsNorm.cs:38-50, ExecuteScalar)."""
    x = x.to(torch.float32)
    mean_sq = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x * (1.0 / torch.sqrt(mean_sq + eps)) * gain


def rope_frequencies(rotary_dim, theta, scaling=None):
    """f_i = theta^(-2i/d) (src/DotLLM.Cpu/Kernels/RoPE.cs:74, FillTables), float64.

    ``scaling`` is config.json's ``rope_scaling`` dict.  For rope_type "llama3":
    wavelengths shorter than P/high keep their frequency, longer than P/low are
    divided by ``factor``, and those between are blended linearly in P/wavelength.
    """
    i = np.arange(rotary_dim // 2, dtype=np.float64)
    freq = 1.0 / np.power(float(theta), 2.0 * i / rotary_dim)
    if scaling is None:
        return freq
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return freq
    if kind != "llama3":
        raise ValueError(f"unsupported rope_scaling type {kind!r}")
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = np.empty_like(freq)
    for n, f in enumerate(freq):
        wavelen = 2.0 * math.pi / f
        if wavelen < orig / high:
            out[n] = f
        elif wavelen > orig / low:
            out[n] = f / factor
        else:
            smooth = (orig / wavelen - low) / (high - low)
            out[n] = (1.0 - smooth) * f / factor + smooth * f
    return out


def rope_tables(positions, rotary_dim, theta, scaling=None):
    """cos/sin of pos * f_i (src/DotLLM.Cpu/Kernels/RoPE.cs:77-85), float64 then float32."""
    freq = rope_frequencies(rotary_dim, theta, scaling)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    return (torch.from_numpy(np.cos(angle).astype(np.float32)),
            torch.from_numpy(np.sin(angle).astype(np.float32)))


def apply_rope(x, cos, sin):
    """Half-split rotation of every head: pairs (x[i], x[i+d/2])
    (src/DotLLM.Cpu/Kernels/RoPE.cs:250-256, ApplyRotationNeoX scalar tail).
    x is [T, heads, head_dim]; cos, sin are [T, d/2] with d <= head_dim."""
    half = cos.shape[-1]
    first = x[..., :half]
    second = x[..., half:2 * half]
    c = cos[:, None, :]
    s = sin[:, None, :]
    out = x.clone()
    out[..., :half] = first * c - second * s
    out[..., half:2 * half] = first * s + second * c
    return out


def causal_attention(q, k, v, n_heads, n_kv_heads, scale, position_offset=0, window=None):
    """Scores, scale, causal (and optional window) mask, softmax, weighted sum
    (src/DotLLM.Cpu/Kernels/Attention.cs:446-519, ExecuteScalar).
    q is [Tq, n_heads*hd]; k and v are [Tk, n_kv_heads*hd]; query i stands at
    position_offset + i and sees keys j <= that (and j > that - window)."""
    tq, tk = q.shape[0], k.shape[0]
    hd = q.shape[1] // n_heads
    group = n_heads // n_kv_heads
    qh = q.view(tq, n_heads, hd)
    kh = k.view(tk, n_kv_heads, hd)
    vh = v.view(tk, n_kv_heads, hd)
    out = torch.empty(tq, n_heads, hd, dtype=torch.float32)
    qi = torch.arange(tq)[:, None] + position_offset
    kj = torch.arange(tk)[None, :]
    hidden = kj > qi
    if window is not None:
        hidden = hidden | (kj < qi - window + 1)
    for h in range(n_heads):
        kvh = h // group
        s = (qh[:, h, :] @ kh[:, kvh, :].T) * scale
        s = s.masked_fill(hidden, float("-inf"))
        s = s - s.max(dim=-1, keepdim=True).values
        w = torch.exp(s)
        w = w / w.sum(dim=-1, keepdim=True)
        out[:, h, :] = w @ vh[:, kvh, :]
    return out.reshape(tq, n_heads * hd)


def swiglu(gate, up):
    """g * sigmoid(g) * u (src/DotLLM.Cpu/Kernels/FusedOps.cs:69-78, SwiGLUScalar)."""
    return gate * (1.0 / (1.0 + torch.exp(-gate))) * up


def linear(x, w):
    """y = x W^T with W [out, in] (src/DotLLM.Cpu/Kernels/MatMul.cs:1121-1134, GemmF32)."""
    return x @ w.T


# ------------------------------------------------------------------ the block
def attention_part(x, weights, prefix, config, cos, sin):
    """Projections, rotation of Q and K, attention, output projection
    (src/DotLLM.Models/Architectures/TransformerModel.cs:235-302)."""
    nh = config["num_attention_heads"]
    nkv = config.get("num_key_value_heads", nh)
    hd = config.get("head_dim") or config["hidden_size"] // nh
    t = x.shape[0]
    q = linear(x, weights[prefix + "self_attn.q_proj.weight"])
    k = linear(x, weights[prefix + "self_attn.k_proj.weight"])
    v = linear(x, weights[prefix + "self_attn.v_proj.weight"])
    q = apply_rope(q.view(t, nh, hd), cos, sin).reshape(t, nh * hd)
    k = apply_rope(k.view(t, nkv, hd), cos, sin).reshape(t, nkv * hd)
    a = causal_attention(q, k, v, nh, nkv, 1.0 / math.sqrt(hd))
    return linear(a, weights[prefix + "self_attn.o_proj.weight"])


def feed_forward_part(x, weights, prefix):
    """down(silu(gate(x)) * up(x)) (TransformerModel.cs:342-382)."""
    g = linear(x, weights[prefix + "mlp.gate_proj.weight"])
    u = linear(x, weights[prefix + "mlp.up_proj.weight"])
    return linear(swiglu(g, u), weights[prefix + "mlp.down_proj.weight"])


def block(h, weights, layer, config, cos, sin):
    """r=h; h=r+attn(norm(h)); r=h; h=r+ffn(norm(h)) (TransformerModel.cs:185-392)."""
    prefix = f"model.layers.{layer}."
    eps = config.get("rms_norm_eps", 1e-5)
    n = rms_norm(h, weights[prefix + "input_layernorm.weight"], eps)
    h = h + attention_part(n, weights, prefix, config, cos, sin)
    n = rms_norm(h, weights[prefix + "post_attention_layernorm.weight"], eps)
    return h + feed_forward_part(n, weights, prefix)


def forward(config, weights, tokens):
    """Logits [T, vocab] of one whole sequence starting at position 0
    (TransformerModel.cs:134-425; the CPU path returns every position)."""
    tokens = list(tokens)
    if len(tokens) > config.get("max_position_embeddings", 2048):
        raise ValueError("sequence longer than max_position_embeddings")
    nh = config["num_attention_heads"]
    hd = config.get("head_dim") or config["hidden_size"] // nh
    cos, sin = rope_tables(range(len(tokens)), hd, config.get("rope_theta", 10000.0),
                           config.get("rope_scaling"))
    h = embed(weights["model.embed_tokens.weight"], tokens)
    for layer in range(config["num_hidden_layers"]):
        h = block(h, weights, layer, config, cos, sin)
    h = rms_norm(h, weights["model.norm.weight"], config.get("rms_norm_eps", 1e-5))
    head = weights["model.embed_tokens.weight"] if config.get("tie_word_embeddings", False) \
        else weights["lm_head.weight"]
    return linear(h, head)


# ------------------------------------------------------------------- sampling
def apply_repetition_penalty(logits, previous, penalty, window):
    """Each distinct id among the last ``window`` generated tokens (0 = all):
    positive logits divided, others multiplied
    (src/DotLLM.Engine/Samplers/RepetitionPenaltyProcessor.cs:14-55)."""
    logits = logits.clone()
    if penalty == 1.0 or not previous:
        return logits
    recent = previous[-window:] if window > 0 else previous
    for tok in sorted(set(recent)):
        if 0 <= tok < logits.numel():
            logits[tok] = logits[tok] / penalty if logits[tok] > 0 else logits[tok] * penalty
    return logits


def apply_temperature(logits, temperature):
    """logits * (1/T), skipped for T<=0 or T==1 (Samplers/TemperatureSampler.cs:22-29)."""
    if temperature <= 0 or temperature == 1.0:
        return logits.clone()
    return logits * torch.tensor(1.0 / temperature, dtype=torch.float32)


def apply_top_k(logits, k):
    """Keep the k largest; ties at the threshold admitted in index order until
    exactly k are kept (Samplers/TopKSampler.cs:32-79)."""
    logits = logits.clone()
    if k <= 0 or k >= logits.numel():
        return logits
    threshold = torch.sort(logits, descending=True).values[k - 1]
    ties_allowed = k - int((logits > threshold).sum())
    for i in range(logits.numel()):
        v = logits[i]
        if v > threshold:
            continue
        if v == threshold and ties_allowed > 0:
            ties_allowed -= 1
            continue
        logits[i] = float("-inf")
    return logits


def softmax(logits):
    """exp(x - max) / sum (src/DotLLM.Cpu/Kernels/Softmax.cs:52-73)."""
    e = torch.exp(logits - logits.max())
    return e / e.sum()


def apply_top_p(logits, p):
    """Smallest set of most probable tokens whose probability sum reaches p
    (Samplers/TopPSampler.cs:23-81).  Among equal probabilities at the cut the
    lower index is kept first (the reference's sort leaves that order open)."""
    logits = logits.clone()
    if p >= 1.0:
        return logits
    probs = softmax(logits)
    order = sorted(range(logits.numel()), key=lambda i: (-float(probs[i]), i))
    total = 0.0
    keep = set()
    for i in order:
        keep.add(i)
        total += float(probs[i])
        if total >= p:
            break
    for i in range(logits.numel()):
        if i not in keep:
            logits[i] = float("-inf")
    return logits


def apply_min_p(logits, min_p):
    """Mask logits below max + ln(min_p) (Samplers/MinPSampler.cs:23-37)."""
    logits = logits.clone()
    if min_p <= 0:
        return logits
    logits[logits < logits.max() + math.log(min_p)] = float("-inf")
    return logits


def categorical(logits, r):
    """First index whose running probability sum exceeds r; argmax as a
    fallback (Samplers/CategoricalSampler.cs:18-41)."""
    probs = softmax(logits)
    total = 0.0
    for i in range(probs.numel()):
        total += float(probs[i])
        if r < total:
            return i
    return int(torch.argmax(probs))


def cdf_interval(logits, index):
    """[lo, hi) of ``index`` on the running probability sum, for tests that accept
    a neighbouring token when r falls within rounding of a boundary."""
    probs = softmax(logits).to(torch.float64)
    lo = float(probs[:index].sum())
    return lo, lo + float(probs[index])


def sample(logits, previous, *, temperature=0.0, top_k=0, top_p=1.0, min_p=0.0,
           repetition_penalty=1.0, repetition_window=0, r=None):
    """Processors, then argmax if greedy, else temperature -> top-k -> top-p ->
    min-p -> categorical (Samplers/SamplerPipeline.cs:141-157, 109-119)."""
    logits = apply_repetition_penalty(logits.to(torch.float32), previous,
                                      repetition_penalty, repetition_window)
    if temperature <= 0:
        return int(torch.argmax(logits))
    logits = apply_temperature(logits, temperature)
    logits = apply_top_k(logits, top_k)
    logits = apply_top_p(logits, top_p)
    logits = apply_min_p(logits, min_p)
    return categorical(logits, r)


def greedy_generate(config, weights, prompt, max_tokens, stop_ids=()):
    """Re-runs the growing sequence without a cache and takes the argmax each time
    (tests/DotLLM.Tests.Integration/Models/Architectures/LlamaForwardPassTests.cs:262-321).
    A stop token ends generation and is not returned (Samplers/StopConditions/EosStopCondition.cs:23-24)."""
    seq = list(prompt)
    out = []
    for _ in range(max_tokens):
        tok = int(torch.argmax(forward(config, weights, seq)[-1]))
        if tok in stop_ids:
            return out, "stop"
        out.append(tok)
        seq.append(tok)
    return out, "length"
