"""Dispatch to the weight-streaming product for steps of a few rows (decode).

The kernel splits k over blocks for matrices with few rows and adds the partial sums through a
scratch buffer; the per-device counter array it synchronises on is kept here.  Launches that
share the counters must be on one stream.
"""
from __future__ import annotations

import torch

from . import library as _library

_P, _I = _library._P, _library._I
_library.register_signatures({
    "dl_gemm_skinny_bf16": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P],
    "dl_gemm_skinny_splits": [_I, _I, _I],
})

MAX_ROWS = 16            # beyond this the library product is used
_MAX_TILES = 1 << 16
_counters = {}
_sms = {}


def _device_state(device):
    key = device.index
    if key not in _counters:
        _counters[key] = torch.zeros(_MAX_TILES, dtype=torch.int32, device=device)
        _sms[key] = _library.library().dl_sm_count()
    return _counters[key], _sms[key]


def takes(x, w, fuse_swiglu=False, max_rows=None):
    M, K = x.shape
    n_out = w.shape[0] // 2 if fuse_swiglu else w.shape[0]
    tiles = (n_out + 7) // 8 if fuse_swiglu else (n_out + 15) // 16
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 1 <= M <= (max_rows or MAX_ROWS)
            and K % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and tiles <= _MAX_TILES)


def run(x, w, out_dtype, fuse_swiglu=False):
    M, K = x.shape
    n_out = w.shape[0] // 2 if fuse_swiglu else w.shape[0]
    counters, sms = _device_state(x.device)
    tiles = (n_out + 7) // 8 if fuse_swiglu else (n_out + 15) // 16
    lib = _library.library()
    ksplit = lib.dl_gemm_skinny_splits(tiles, K, sms)
    nt = 1 if M <= 8 else 2 if M <= 16 else 4 if M <= 32 else 8
    partials = torch.empty(tiles * ksplit * nt * 128, dtype=torch.float32, device=x.device) if ksplit > 1 else None
    out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    _library.call("dl_gemm_skinny_bf16", x.data_ptr(), x.stride(0) if M > 1 else max(K, x.stride(0)),
                  w.data_ptr(), out.data_ptr(), 0 if out_dtype == torch.float32 else 1, n_out, M, n_out, K,
                  1 if fuse_swiglu else 0, ksplit, None if partials is None else partials.data_ptr(),
                  counters.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return out


def maybe_run(x, w, out_dtype, fuse_swiglu=False):
    """y = x W^T (or the gated form) by the skinny kernel when it takes the sizes, else None."""
    if not takes(x, w, fuse_swiglu):
        return None
    return run(x, w, out_dtype, fuse_swiglu)
