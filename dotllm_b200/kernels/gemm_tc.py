"""Dispatch to the tcgen05 product for steps of many rows (prefill).

Used where fusing pays: the gate/up projection with the SwiGLU gating in the epilogue, and a prompt's
Q/K/V projection with the rotation and the cache write in the epilogue.  The plain product is available
too (tests and the microbenchmark compare it with the library's).
"""
from __future__ import annotations

import torch

from . import library as _library

_P, _I = _library._P, _library._I
_library.register_signatures({
    "dl_gemm_tc_bf16": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "dl_gemm_tc_qkv_bf16": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _I, _P, _P, _P, _I, _P, _P, _I, _I, _P, _P],
})

MIN_ROWS = 17            # fewer rows go to the weight-streaming kernel
BLOCKS = 0               # > 0: persistent blocks (tuning and tests); 0: one per multiprocessor
QKV_MIN_ROWS = 129       # a prompt step: fewer rows are a decode step's (rotation and cache write inside the attention kernel)
# True: a prompt's Q/K/V product rotates and writes the cache in its epilogue (same bits).  Off: the
# tcgen05 product is slower than the library's at that shape by more than the rope and cache-write
# kernel costs (2,048 x 4,096 x 6,144: 95 us against 73.6 + 13.9).
QKV_FUSED = False


def takes(x, w, fuse_swiglu=False):
    M, K = x.shape
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and M >= MIN_ROWS and K % 8 == 0
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.stride(0) >= K and x.data_ptr() % 16 == 0
            and w.is_contiguous() and w.data_ptr() % 16 == 0 and (not fuse_swiglu or w.shape[0] % 2 == 0))


def run(x, w, out_dtype, fuse_swiglu=False):
    M, K = x.shape
    n_out = w.shape[0] // 2 if fuse_swiglu else w.shape[0]
    out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    _library.call("dl_gemm_tc_bf16", x.data_ptr(), x.stride(0), w.data_ptr(), out.data_ptr(),
                  0 if out_dtype == torch.float32 else 1, n_out, M, n_out, K, 1 if fuse_swiglu else 0, BLOCKS,
                  _library.status_word(x.device).data_ptr(), _library.current_stream())
    return out


def takes_qkv(x, w, q_cols, kv_cols, head_dim, rotary_dim, cos, sin, k_pool, v_pool):
    """Can the Q/K/V product of these rows rotate and write the cache in its epilogue?"""
    if not QKV_FUSED or not isinstance(x, torch.Tensor) or x.dim() != 2 or x.shape[0] < QKV_MIN_ROWS:
        return False
    return (takes(x, w) and head_dim in (64, 128) and rotary_dim == head_dim and q_cols % 256 == 0 and kv_cols % 256 == 0
            and w.shape[0] == q_cols + 2 * kv_cols and cos is not None and cos.dtype == torch.float32
            and cos.is_contiguous() and sin.is_contiguous() and cos.data_ptr() % 16 == 0 and sin.data_ptr() % 16 == 0
            and k_pool.dtype == torch.bfloat16 and v_pool.dtype == torch.bfloat16)


def run_qkv(x, w, q_cols, kv_cols, head_dim, n_kv_heads, cos, sin, token_pos, token_seq, block_table, k_pool, v_pool):
    """The rotated queries [M, q_cols]; the rotated keys and the values are in the cache when the kernel is done."""
    M, K = x.shape
    q = torch.empty((M, q_cols), dtype=torch.bfloat16, device=x.device)
    _library.call("dl_gemm_tc_qkv_bf16", x.data_ptr(), x.stride(0), w.data_ptr(), q.data_ptr(), q_cols, M, K, q_cols, kv_cols,
                  head_dim, n_kv_heads, cos.data_ptr(), sin.data_ptr(), cos.shape[0], token_pos.data_ptr(), token_seq.data_ptr(),
                  block_table.data_ptr(), block_table.shape[1], k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0], BLOCKS,
                  _library.status_word(x.device).data_ptr(), _library.current_stream())
    return q
