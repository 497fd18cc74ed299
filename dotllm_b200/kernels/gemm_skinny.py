"""Dispatch to the weight-streaming products for steps of a few rows (decode).

Up to ``SKINNY_ROWS`` rows go to the mma.sync kernel of csrc/gemm_skinny.cu (it can take 16), more, up
to 128, to the tcgen05 kernel of csrc/gemm_decode_tc.cu (``gemm_decode_tc.run``, same contract).  The first cuts its work into
equal shares per warp; tiles that straddle two shares are summed through a scratch buffer with
arrival counters.  Both are kept here per device (they are small and every launch leaves the
counters zero).  Launches that share them must be on one stream.
"""
from __future__ import annotations

import ctypes

import torch

from . import gemm_decode_tc
from . import library as _library

_P, _I, _F = _library._P, _library._I, _library._F
_library.register_signatures({
    "dl_gemm_skinny_bf16": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P, _I, _P, _I, _P, _P],
    "dl_gemm_skinny_fused_bf16": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P, _I, _P, _P, _I, _F, _F,
                                  _P, _I, _P, _I, _P, _P],
    "dl_gemm_skinny_scratch": [_I, _I, _I, _I, _I, _P, _P],
})

KERNEL_ROWS = 16         # rows the mma.sync kernel can take (two tiles of eight)
# Rows up to which the dispatcher gives a product to the mma.sync kernel; more go the way of 17 and
# more (the gated product to the tcgen05 kernel, the plain ones to the library).  Measured on whole
# decode steps at the 8B shape: 9 rows 4.76 against 4.79 ms, 12 rows 5.30 against 5.24, 16 rows 6.08
# against 5.83 - the second tile of eight rows costs the mma.sync kernel more than the library's
# launch costs the step.
SKINNY_ROWS = 10
MAX_ROWS = 128           # rows the two kernels take between them; beyond this the products are prefill products
# Of 17 to 128 rows the gated product goes to the tcgen05 kernel (47 us against 56 for the library product plus
# gating at the 8B shape and 64 rows).  The plain products do too when TC_PLAIN is set; measured inside a decode
# step the library's are about 7 us a product faster at those sizes, so they stay with the library.
TC_PLAIN = False
SUM_STRIDE = 16          # floats between the sums of squares of two 16-column tiles (mma.sync kernel)
_MAX_TILES = 1 << 16
_state = {}


def _device_state(device):
    key = device.index
    if key not in _state:
        sms = _library.library().dl_sm_count()
        counters = torch.zeros(_MAX_TILES, dtype=torch.int32, device=device)
        _library.register_counters(counters)
        partials = torch.empty(max(sms, 1) * 6 * 2 * 2 * 128, dtype=torch.float32, device=device)
        _state[key] = (counters, partials, sms)
    return _state[key]


def sum_stride(rows):
    """Floats between two parts of the sums of squares that a product of ``rows`` rows leaves."""
    return SUM_STRIDE if rows <= SKINNY_ROWS else gemm_decode_tc.SUM_STRIDE


def takes(x, w, fuse_swiglu=False, max_rows=None):
    M, K = x.shape
    if M > SKINNY_ROWS:
        return (fuse_swiglu or TC_PLAIN) and M <= (max_rows or MAX_ROWS) and gemm_decode_tc.takes(x, w, fuse_swiglu)
    n_out = w.shape[0] // 2 if fuse_swiglu else w.shape[0]
    tiles = (n_out + 7) // 8 if fuse_swiglu else (n_out + 15) // 16
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and 1 <= M <= min(MAX_ROWS, max_rows or MAX_ROWS)
            and K % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and tiles <= _MAX_TILES)


def run(x, w, out_dtype, fuse_swiglu=False, resident=False, row_sums=None, into=None):
    """``row_sums`` = (sums float32 [parts * 16], parts, width, eps): x is a stream times a norm's gain,
    and every output row is multiplied by rsqrt(sum of the row's parts / width + eps); the sums must come
    from a product of the same number of rows (``sum_stride``).
    ``into`` = (stream float32 [M, N], gain float32 [N]): the product is added into the stream in place;
    returns (stream * gain as bfloat16 [M, N], sums of squares float32 [ceil(N / 16) * 16])."""
    M, K = x.shape
    if M > SKINNY_ROWS:
        return gemm_decode_tc.run(x, w, out_dtype, fuse_swiglu, resident, row_sums, into)
    n_out = w.shape[0] // 2 if fuse_swiglu else w.shape[0]
    counters, partials, sms = _device_state(x.device)
    x_stride = x.stride(0) if M > 1 else max(K, x.stride(0))
    flags = (1 if fuse_swiglu else 0) | (2 if resident else 0)
    tail = (partials.data_ptr(), partials.numel(), counters.data_ptr(), counters.numel(),
            _library.status_word(x.device).data_ptr(), _library.current_stream())
    if row_sums is None and into is None:
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
        _library.call("dl_gemm_skinny_bf16", x.data_ptr(), x_stride, w.data_ptr(), out.data_ptr(),
                      0 if out_dtype == torch.float32 else 1, n_out, M, n_out, K, flags, *tail)
        return out
    sums_in, parts, width, eps = row_sums if row_sums is not None else (None, 0, 1, 0.0)
    if into is not None:
        stream, gain = into
        scaled = torch.empty((M, n_out), dtype=torch.bfloat16, device=x.device)
        sums_out = torch.empty(((n_out + 15) // 16) * 16, dtype=torch.float32, device=x.device)
        out, out_stride, result = stream, stream.stride(0), (scaled, sums_out)
    else:
        gain = scaled = sums_out = None
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
        out_stride, result = n_out, out
    _library.call("dl_gemm_skinny_fused_bf16", x.data_ptr(), x_stride, w.data_ptr(), out.data_ptr(),
                  0 if out.dtype == torch.float32 else 1, out_stride, M, n_out, K, flags,
                  gain.data_ptr() if gain is not None else None, scaled.data_ptr() if scaled is not None else None, n_out,
                  sums_out.data_ptr() if sums_out is not None else None,
                  sums_in.data_ptr() if sums_in is not None else None, parts, 1.0 / width, float(eps), *tail)
    return result


def scratch_need(M, N, K, fuse_swiglu=False, sms=148):
    """(partial floats, counters) the product of these sizes needs."""
    a, b = ctypes.c_int(0), ctypes.c_int(0)
    _library.library().dl_gemm_skinny_scratch(M, N, K, 1 if fuse_swiglu else 0, sms, ctypes.byref(a), ctypes.byref(b))
    return a.value, b.value


def maybe_run(x, w, out_dtype, fuse_swiglu=False, resident=False):
    """y = x W^T (or the gated form) by the skinny kernel when it takes the sizes, else None.
    ``resident``: no work still pending on the stream writes W."""
    if not takes(x, w, fuse_swiglu):
        return None
    return run(x, w, out_dtype, fuse_swiglu, resident)
