"""Dispatch to the tensor-core attention kernels for the sizes they take.

Decode steps (one new token per sequence) go to the split-key kernel of csrc/attention_decode.cu.
Its scratch (per-run partial sums) is allocated once per step and shared by the layers, which run
one after another on one stream; the counters it synchronises on are kept per device.
"""
from __future__ import annotations

import torch

from . import library as _library

_P, _I, _F = _library._P, _library._I, _library._F
_library.register_signatures({
    "dl_attention_decode_bf16": [_P, _I, _P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I,
                                 _P, _P, _P, _P],
    "dl_attention_prefill_bf16": [_P, _I, _P, _I, _P, _P, _I, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I,
                                  _F, _I, _P, _P],
})

PREFILL_ROWS = 128       # query rows per block of the prefill kernel (AP_ROWS)

DECODE_HEAD_DIMS = (32, 64, 96, 128)
RUNS_PER_BLOCK = 0       # > 0: force this many runs per persistent decode block (tuning and tests)


def keys_per_split(longest, pairs, sms=148):
    """Keys in one run of a (sequence, KV head).  The decode kernel is persistent, one block per
    multiprocessor taking runs in turn: several runs per block even out the load, runs of a few
    pages keep all of a block's warps busy.  ``pairs`` is sequences x KV heads."""
    if RUNS_PER_BLOCK:                       # explicit override (tuning and tests)
        want_splits = max(1, (RUNS_PER_BLOCK * sms + pairs - 1) // pairs)
        kps = (longest + want_splits - 1) // want_splits
        return max(128, min(2048, (kps + 63) // 64 * 64))
    # Cost model: blocks work in rounds of `sms` runs; a run costs its pages plus about three pages'
    # worth of start-up and merging.  Pick the run length with the cheapest total.
    best, best_cost = 2048, None
    pages_total = (longest + 63) // 64
    for pages in range(2, min(32, pages_total) + 1):
        n_splits = (pages_total + pages - 1) // pages
        rounds = (pairs * n_splits + sms - 1) // sms
        cost = rounds * (pages + 3)
        if best_cost is None or cost < best_cost or (cost == best_cost and pages * 64 > best):
            best, best_cost = pages * 64, cost
    return best


def decode_fits(group, head_dim):
    """Whether at least two ring stages and the merge buffers of the decode kernel fit in shared
    memory (it takes up to six stages when they fit)."""
    return 2 * 2 * 64 * head_dim * 2 + 4 * group * (head_dim + 4) * 4 + 4096 <= 227 * 1024


def _decode(q, q_stride, out, k_pool, v_pool, n_pages, block_table, n_heads, n_kv_heads, head_dim,
            scale, window, plan):
    B = plan.n_seqs
    group = n_heads // n_kv_heads
    longest = min(plan.max_total, window + 64) if window else plan.max_total
    kps = keys_per_split(longest, B * n_kv_heads)
    max_splits = max(1, (longest + kps - 1) // kps)
    key = ("decode", n_kv_heads, group, head_dim, max_splits)
    if key not in plan.scratch:
        plan.scratch[key] = (
            torch.empty(B * n_kv_heads * max_splits * group * head_dim, dtype=torch.float32, device=q.device),
            torch.empty(B * n_kv_heads * max_splits * group * 2, dtype=torch.float32, device=q.device))
    part_o, part_ml = plan.scratch[key]
    _library.call("dl_attention_decode_bf16", q.data_ptr(), q_stride, out.data_ptr(), out.stride(0),
                  k_pool.data_ptr(), v_pool.data_ptr(), n_pages, plan.seq_total.data_ptr(),
                  block_table.data_ptr(), block_table.shape[1], B, n_heads, n_kv_heads, head_dim,
                  scale, window, kps, max_splits, part_o.data_ptr(), part_ml.data_ptr(),
                  _library.status_word(q.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    return True


def _prefill(q, q_stride, out, k_pool, v_pool, n_pages, block_table, n_heads, n_kv_heads, head_dim,
             scale, window, plan):
    if "prefill_tiles" not in plan.scratch:
        tile_seq, tile_row0 = [], []
        for b, n in enumerate(plan.news):
            for r0 in range(0, n, PREFILL_ROWS):
                tile_seq.append(b)
                tile_row0.append(r0)
        host = torch.tensor(tile_seq + tile_row0, dtype=torch.int32)
        dev = host.pin_memory().to(q.device, non_blocking=True)
        plan.scratch["prefill_tiles"] = (dev[:len(tile_seq)], dev[len(tile_seq):], len(tile_seq))
    tile_seq, tile_row0, n_tiles = plan.scratch["prefill_tiles"]
    _library.call("dl_attention_prefill_bf16", q.data_ptr(), q_stride, out.data_ptr(), out.stride(0),
                  k_pool.data_ptr(), v_pool.data_ptr(), n_pages, tile_seq.data_ptr(), tile_row0.data_ptr(),
                  n_tiles, plan.seq_start.data_ptr(), plan.seq_new.data_ptr(), plan.cu_new.data_ptr(),
                  block_table.data_ptr(), block_table.shape[1], n_heads, n_kv_heads, head_dim, scale, window,
                  _library.status_word(q.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    return True


def run(q, q_stride, out, k_pool, v_pool, n_pages, token_seq, token_pos, block_table,
        n_heads, n_kv_heads, head_dim, scale, window, plan):
    """Run a tensor-core kernel into ``out`` and return True, or return False to let the
    generic kernel take the call."""
    if q.dtype != torch.bfloat16 or q_stride % 8 or q.data_ptr() % 16 or head_dim not in DECODE_HEAD_DIMS:
        return False
    if plan.all_single and q.shape[0] == plan.n_seqs:
        if n_heads // n_kv_heads > 16 or not decode_fits(n_heads // n_kv_heads, head_dim):
            return False
        return _decode(q, q_stride, out, k_pool, v_pool, n_pages, block_table, n_heads, n_kv_heads,
                       head_dim, scale, window, plan)
    if plan.news and q.shape[0] == sum(plan.news):
        return _prefill(q, q_stride, out, k_pool, v_pool, n_pages, block_table, n_heads, n_kv_heads,
                        head_dim, scale, window, plan)
    return False
