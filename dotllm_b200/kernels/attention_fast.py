"""Dispatch to the tensor-core attention kernels for the sizes they take.

Decode steps (one new token per sequence) go to the stream-K kernel of csrc/attention_decode.cu,
which cuts the step's cache pages into equal shares per block on the device.  Its scratch (the
partial results of cut segments, two per block) is allocated once per step and shared by the
layers, which run one after another on one stream.
"""
from __future__ import annotations

import torch

from . import library as _library

_P, _I, _F = _library._P, _library._I, _library._F
_library.register_signatures({
    "dl_attention_decode_bf16": [_P, _I, _P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I,
                                 _P, _P, _I, _P, _I, _P, _P],
    "dl_attention_decode_fresh_bf16": [_P, _I, _P, _I, _P, _I, _P, _P, _I, _I, _P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I,
                                       _I, _F, _I, _I, _P, _P, _I, _P, _I, _P, _P],
    "dl_attention_prefill_bf16": [_P, _I, _P, _I, _P, _P, _I, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I,
                                  _F, _I, _P, _P],
    "dl_attention_prefill_tc_bf16": [_P, _I, _I, _P, _I, _P, _P, _I, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I,
                                     _F, _I, _P, _P],
})

PREFILL_ROWS = 128       # query rows per block of the mma.sync prefill kernel (AP_ROWS)
PREFILL_TC_ROWS = 256    # ... and of the tcgen05 one (PT_TILES * PT_ROWS)
PREFILL_TC_HEAD_DIMS = (64, 128)     # head sizes of the tcgen05 prefill kernel; others take the mma.sync one
PREFILL_TC = True        # False: always the mma.sync kernel (tests compare the two)

DECODE_HEAD_DIMS = (32, 64, 96, 128)
DECODE_BLOCKS = 0        # > 0: persistent blocks of the decode kernel (tuning and tests); 0: one per multiprocessor


def decode_fits(group, head_dim):
    """Whether at least two ring stages and the merge buffers of the decode kernel fit in shared
    memory (it takes up to six stages when they fit)."""
    return 2 * 2 * 64 * head_dim * 2 + 4 * group * (head_dim + 4) * 4 + 4096 <= 227 * 1024


def _decode(q, q_stride, out, k_pool, v_pool, n_pages, block_table, n_heads, n_kv_heads, head_dim,
            scale, window, plan):
    B = plan.n_seqs
    group = n_heads // n_kv_heads
    part_o, part_ml, slots = _decode_scratch(plan, group, head_dim, q.device)
    counters = _pair_counters(q.device)
    _library.call("dl_attention_decode_bf16", q.data_ptr(), q_stride, out.data_ptr(), out.stride(0),
                  k_pool.data_ptr(), v_pool.data_ptr(), n_pages, plan.seq_total.data_ptr(),
                  block_table.data_ptr(), block_table.shape[1], B, n_heads, n_kv_heads, head_dim,
                  scale, window, DECODE_BLOCKS, part_o.data_ptr(), part_ml.data_ptr(), slots,
                  counters.data_ptr(), counters.numel(),
                  _library.status_word(q.device).data_ptr(), _library.current_stream())
    return True


_counters = {}


def _pair_counters(device):
    """Per device: one arrival counter per (sequence, KV head) of a decode step.  Zero at rest: the block
    that finishes a pair resets its counter.  Launches that share them must be on one stream."""
    key = device.index
    if key not in _counters:
        _counters[key] = torch.zeros(1 << 16, dtype=torch.int32, device=device)
        _library.register_counters(_counters[key])
    return _counters[key]


def _decode_scratch(plan, group, head_dim, device):
    slots = 2 * max(1, _library.library().dl_sm_count())
    key = ("decode", group, head_dim)
    if key not in plan.scratch:
        plan.scratch[key] = (torch.empty(slots * group * head_dim, dtype=torch.float32, device=device),
                             torch.empty(slots * group * 2, dtype=torch.float32, device=device))
    return plan.scratch[key] + (slots,)


FRESH_ROTATE_HEAD_DIMS = (64, 128)   # head sizes whose rotation the decode kernel does itself


def decode_fresh(q, k, v, cos, sin, rotary_dim, block_table, k_pool, v_pool, n_heads, n_kv_heads, head_dim,
                 scale, window, plan):
    """A decode step with the new token handled inside the attention kernel (rotation of q and k,
    cache write, attention): returns the output, or None when the sizes are not the kernel's."""
    group = n_heads // n_kv_heads
    if not (plan.all_single and q.shape[0] == plan.n_seqs and head_dim in DECODE_HEAD_DIMS and group <= 16
            and decode_fits(group, head_dim) and (rotary_dim == 0 or (rotary_dim == head_dim
                                                                      and head_dim in FRESH_ROTATE_HEAD_DIMS))):
        return None
    rows = lambda t: t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])
    qs, ks, vs = rows(q), rows(k), rows(v)
    if q.stride(1) != 1 or k.stride(1) != 1 or v.stride(1) != 1 or qs % 8 or ks % 4 or vs % 4 \
            or q.data_ptr() % 16 or k.data_ptr() % 8 or v.data_ptr() % 8 or k.dtype != q.dtype or v.dtype != q.dtype \
            or k_pool.dtype != q.dtype or v_pool.dtype != q.dtype:
        return None
    if rotary_dim and (cos.dtype != torch.float32 or sin.dtype != torch.float32 or not cos.is_contiguous()
                       or not sin.is_contiguous() or cos.shape != sin.shape or cos.shape[1] != head_dim // 2
                       or cos.data_ptr() % 16 or sin.data_ptr() % 16):
        return None
    B = plan.n_seqs
    out = torch.empty((B, n_heads * head_dim), dtype=q.dtype, device=q.device)
    part_o, part_ml, slots = _decode_scratch(plan, group, head_dim, q.device)
    counters = _pair_counters(q.device)
    _library.call("dl_attention_decode_fresh_bf16", q.data_ptr(), qs, k.data_ptr(), ks, v.data_ptr(), vs,
                  cos.data_ptr() if rotary_dim else None, sin.data_ptr() if rotary_dim else None,
                  cos.shape[0] if rotary_dim else 0, 1 if rotary_dim else 0, out.data_ptr(), out.stride(0),
                  k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0], plan.seq_total.data_ptr(),
                  block_table.data_ptr(), block_table.shape[1], B, n_heads, n_kv_heads, head_dim, scale, window,
                  DECODE_BLOCKS, part_o.data_ptr(), part_ml.data_ptr(), slots, counters.data_ptr(), counters.numel(),
                  _library.status_word(q.device).data_ptr(), _library.current_stream())
    return out


def _prefill(q, q_stride, out, k_pool, v_pool, n_pages, block_table, n_heads, n_kv_heads, head_dim,
             scale, window, plan):
    tc = PREFILL_TC and head_dim in PREFILL_TC_HEAD_DIMS and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0
    rows = PREFILL_TC_ROWS if tc else PREFILL_ROWS
    if ("prefill_tiles", rows) not in plan.scratch:
        # tiles that see the most keys first: the kernels start blocks in this order, and the short
        # ones at the end fill the multiprocessors' last gaps
        tiles = [(b, r0) for b, n in enumerate(plan.news) for r0 in range(0, n, rows)]
        tiles.sort(key=lambda t: -(plan.starts[t[0]] + min(plan.news[t[0]], t[1] + rows)))
        tile_seq, tile_row0 = [t[0] for t in tiles], [t[1] for t in tiles]
        host = torch.tensor(tile_seq + tile_row0, dtype=torch.int32).pin_memory()
        dev = host.to(q.device, non_blocking=True)
        # the pinned list stays with the plan: a captured step copies it again, from this memory, at every replay
        plan.scratch[("prefill_tiles", rows)] = (dev[:len(tile_seq)], dev[len(tile_seq):], len(tile_seq), host)
    tile_seq, tile_row0, n_tiles, _ = plan.scratch[("prefill_tiles", rows)]
    if tc:
        _library.call("dl_attention_prefill_tc_bf16", q.data_ptr(), q_stride, q.shape[0], out.data_ptr(), out.stride(0),
                      k_pool.data_ptr(), v_pool.data_ptr(), n_pages, tile_seq.data_ptr(), tile_row0.data_ptr(),
                      n_tiles, plan.seq_start.data_ptr(), plan.seq_new.data_ptr(), plan.cu_new.data_ptr(),
                      block_table.data_ptr(), block_table.shape[1], n_heads, n_kv_heads, head_dim, scale, window,
                      _library.status_word(q.device).data_ptr(), _library.current_stream())
        return True
    _library.call("dl_attention_prefill_bf16", q.data_ptr(), q_stride, out.data_ptr(), out.stride(0),
                  k_pool.data_ptr(), v_pool.data_ptr(), n_pages, tile_seq.data_ptr(), tile_row0.data_ptr(),
                  n_tiles, plan.seq_start.data_ptr(), plan.seq_new.data_ptr(), plan.cu_new.data_ptr(),
                  block_table.data_ptr(), block_table.shape[1], n_heads, n_kv_heads, head_dim, scale, window,
                  _library.status_word(q.device).data_ptr(), _library.current_stream())
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
