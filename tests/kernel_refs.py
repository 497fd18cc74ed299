"""Plain torch references of every kernel wrapper in ``dotllm_b200.kernels.ops``, with the same
signatures, on whatever device the tensors live on.

Two uses: each CUDA kernel is compared with its function here, alone and at sizes the engine
does not use; and the CPU tests swap these in for the CUDA wrappers to exercise the engine's
host logic.  Arithmetic is float32 (float64 where it is free); results are rounded to the dtype
the kernel writes.  Formulas as in tests/plain_llama.py, which cites the reference.
"""
from __future__ import annotations

import torch

import plain_llama

PAGE = 64


def gather_rows(table, ids, out=None, out_dtype=torch.float32):
    res = table[ids.long()].to(out_dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


def add_rmsnorm(residual, delta, gain, eps, out_dtype, lazy=False):
    if delta is not None:
        residual += delta.to(torch.float32)
    return plain_llama.rms_norm(residual, gain, eps).to(out_dtype)


def _rotate(x, cos, sin, positions, n_heads, head_dim, rotary_dim):
    t = x.shape[0]
    xf = x.to(torch.float32).reshape(t, n_heads, head_dim)
    c, s = cos[positions.long()], sin[positions.long()]
    return plain_llama.apply_rope(xf, c, s).reshape(t, n_heads * head_dim)


def rope_cache_write(q, k, v, cos, sin, rotary_dim, token_seq, token_pos, block_table,
                     k_pool, v_pool, n_heads, n_kv_heads, head_dim, write_cache=True):
    if rotary_dim:
        q.copy_(_rotate(q, cos, sin, token_pos, n_heads, head_dim, rotary_dim).to(q.dtype))
    if not write_cache:
        return
    kr = _rotate(k, cos, sin, token_pos, n_kv_heads, head_dim, rotary_dim).to(k.dtype) if rotary_dim else k
    for t in range(q.shape[0]):
        pos = int(token_pos[t])
        page = int(block_table[int(token_seq[t]), pos // PAGE])
        assert page >= 0
        k_pool[page, :, pos % PAGE, :] = kr[t].reshape(n_kv_heads, head_dim)
        v_pool[page, :, :, pos % PAGE] = v[t].reshape(n_kv_heads, head_dim)


def gather_kv(k_pool, v_pool, pages, length):
    """Keys and values [length, nkv, hd] of one sequence from its pages (float32)."""
    ks, vs = [], []
    for j in range(length):
        page = int(pages[j // PAGE])
        ks.append(k_pool[page, :, j % PAGE, :])
        vs.append(v_pool[page, :, :, j % PAGE])
    return torch.stack(ks).to(torch.float32), torch.stack(vs).to(torch.float32)


def attention(q, k_pool, v_pool, token_seq, token_pos, block_table, n_heads, n_kv_heads,
              head_dim, scale, window=0, plan=None, score_hook=None):
    if score_hook:
        return _attention_with_hook(q, k_pool, v_pool, token_seq, token_pos, block_table, n_heads, n_kv_heads, head_dim,
                                    scale, window, score_hook)
    T = q.shape[0]
    out = torch.empty((T, n_heads * head_dim), dtype=torch.float32, device=q.device)
    for t in range(T):
        pos = int(token_pos[t])
        first = max(0, pos - window + 1) if window else 0
        pages = block_table[int(token_seq[t])]
        ks, vs = [], []
        for j in range(first, pos + 1):
            page = int(pages[j // PAGE])
            ks.append(k_pool[page, :, j % PAGE, :])
            vs.append(v_pool[page, :, :, j % PAGE])
        k = torch.stack(ks).to(torch.float32).reshape(len(ks), n_kv_heads * head_dim)
        v = torch.stack(vs).to(torch.float32).reshape(len(vs), n_kv_heads * head_dim)
        # one query at the last of these keys: the causal mask hides nothing
        out[t] = plain_llama.causal_attention(q[t:t + 1].to(torch.float32), k, v, n_heads, n_kv_heads,
                                              scale, position_offset=len(ks) - 1)[0]
    return out.to(q.dtype)


def _attention_with_hook(q, k_pool, v_pool, token_seq, token_pos, block_table, n_heads, n_kv_heads, head_dim, scale,
                         window, hook):
    """Scores capped (softcap * tanh(s / softcap)) and then biased by slope * (key - query position)."""
    T = q.shape[0]
    out = torch.empty((T, n_heads * head_dim), dtype=torch.float32, device=q.device)
    group = n_heads // n_kv_heads
    for t in range(T):
        pos = int(token_pos[t])
        first = max(0, pos - window + 1) if window else 0
        k, v = gather_kv(k_pool, v_pool, block_table[int(token_seq[t])], pos + 1)
        for h in range(n_heads):
            qh = q[t, h * head_dim:(h + 1) * head_dim].to(torch.float32)
            s = (k[first:, h // group] @ qh) * scale
            if hook.softcap > 0:
                s = hook.softcap * torch.tanh(s / hook.softcap)
            if hook.slopes is not None:
                s = s + float(hook.slopes[h]) * (torch.arange(first, pos + 1, dtype=torch.float32) - pos)
            w = torch.softmax(s, dim=0)
            out[t, h * head_dim:(h + 1) * head_dim] = w @ v[first:, h // group]
    return out.to(q.dtype)


def swiglu(gate_up):
    i = gate_up.shape[1] // 2
    g, u = gate_up[:, :i].to(torch.float32), gate_up[:, i:].to(torch.float32)
    return plain_llama.swiglu(g, u).to(gate_up.dtype)


def linear(x, w, out_dtype=None, resident=False, lazy=False):
    y = x.to(torch.float32) @ w.to(torch.float32).T
    return y.to(out_dtype or x.dtype)


def gated_linear(x, w_gate_up, resident=False):
    return swiglu(linear(x, w_gate_up, torch.float32)).to(x.dtype)


def repetition_penalty(logits, prev, prev_len, penalty, window, row_map=None, append=None):
    for r in range(logits.shape[0]):
        h = int(row_map[r]) if row_map is not None else r
        if append is not None and int(append[0][r]) >= 0:
            prev[h, int(append[0][r])] = int(append[1][r])
        previous = prev[h, :int(prev_len[r])].tolist()
        logits[r] = plain_llama.apply_repetition_penalty(logits[r].cpu(), previous, float(penalty[r]),
                                                         int(window[r])).to(logits.device)
    return logits


def sample(logits, temperature=None, top_k=None, top_p=None, min_p=None, uniform=None, out=None, split=None):
    out = []
    for r in range(logits.shape[0]):
        row = logits[r].detach().cpu()
        t = float(temperature[r]) if temperature is not None else 0.0
        out.append(plain_llama.sample(
            row, [], temperature=t, top_k=int(top_k[r]) if top_k is not None else 0,
            top_p=float(top_p[r]) if top_p is not None else 1.0,
            min_p=float(min_p[r]) if min_p is not None else 0.0,
            r=float(uniform[r]) if uniform is not None else None))
    return torch.tensor(out, dtype=torch.int32, device=logits.device)
