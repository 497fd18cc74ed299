"""Dispatch to the tcgen05 weight-streaming product for decode steps of 17 to 128 rows.

The kernel cuts its work into equal shares per block; a tile of W that straddles two shares is
summed through a scratch buffer with arrival counters.  Both are kept here per device (the counters
are zero between launches; the partial sums are sized for the largest product).  Launches that share
them must be on one stream.
"""
from __future__ import annotations

import ctypes

import torch

from . import library as _library

_P, _I, _F, _L = _library._P, _library._I, _library._F, ctypes.c_longlong
_library.register_signatures({
    "dl_gemm_decode_tc_bf16": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P, _I, _P, _P, _I, _F, _F,
                               _P, _L, _P, _I, _P, _P],
    "dl_gemm_decode_tc_scratch": [_I, _I, _I, _I, _I, _P, _P],
})

MAX_ROWS = 128           # rows the kernel takes
SUM_STRIDE = 128         # floats between the sums of squares of two 128-column tiles
_MAX_TILES = 1 << 14
_state = {}


def scratch_need(M, N, K, gated=False, sms=148):
    """(partial floats, counters) the product of these sizes needs."""
    a, b = ctypes.c_longlong(0), ctypes.c_int(0)
    _library.library().dl_gemm_decode_tc_scratch(M, N, K, 1 if gated else 0, sms, ctypes.byref(a), ctypes.byref(b))
    return a.value, b.value


def _device_state(device):
    key = device.index
    if key not in _state:
        sms = _library.library().dl_sm_count()
        counters = torch.zeros(_MAX_TILES, dtype=torch.int32, device=device)
        _library.register_counters(counters)
        # Two parts per block of at most 256 accumulator columns by 128 outputs: the largest product
        # (128 rows, gated) fits, so the buffer never moves under a captured graph.
        partials = torch.empty(max(sms, 1) * 2 * 256 * 128, dtype=torch.float32, device=device)
        _state[key] = (counters, partials)
    return _state[key]


def takes(x, w, gated=False):
    M, K = x.shape
    n_out = w.shape[0] // 2 if gated else w.shape[0]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 1 <= M <= MAX_ROWS
            and K % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.is_contiguous() and w.data_ptr() % 16 == 0 and (n_out + 127) // 128 <= _MAX_TILES)


def run(x, w, out_dtype, fuse_swiglu=False, resident=False, row_sums=None, into=None):
    """Same contract as ``gemm_skinny.run``; sums of squares are laid out [tile of 128 columns][128]."""
    M, K = x.shape
    n_out = w.shape[0] // 2 if fuse_swiglu else w.shape[0]
    counters, partials = _device_state(x.device)
    x_stride = x.stride(0) if M > 1 else max(K, x.stride(0))
    flags = (1 if fuse_swiglu else 0) | (2 if resident else 0)
    sums_in, parts, width, eps = row_sums if row_sums is not None else (None, 0, 1, 0.0)
    if into is not None:
        stream, gain = into
        scaled = torch.empty((M, n_out), dtype=torch.bfloat16, device=x.device)
        sums_out = torch.empty(((n_out + 127) // 128) * SUM_STRIDE, dtype=torch.float32, device=x.device)
        out, out_stride, result = stream, stream.stride(0), (scaled, sums_out)
    else:
        gain = scaled = sums_out = None
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
        out_stride, result = n_out, out
    _library.call("dl_gemm_decode_tc_bf16", x.data_ptr(), x_stride, w.data_ptr(), out.data_ptr(),
                  0 if out.dtype == torch.float32 else 1, out_stride, M, n_out, K, flags,
                  gain.data_ptr() if gain is not None else None, scaled.data_ptr() if scaled is not None else None, n_out,
                  sums_out.data_ptr() if sums_out is not None else None,
                  sums_in.data_ptr() if sums_in is not None else None, parts, 1.0 / width, float(eps),
                  partials.data_ptr(), partials.numel(), counters.data_ptr(), counters.numel(),
                  _library.status_word(x.device).data_ptr(), _library.current_stream())
    return result
