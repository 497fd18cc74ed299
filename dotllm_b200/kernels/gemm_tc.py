"""Dispatch to the tcgen05 product for steps of many rows (prefill).

Used where fusing pays: the gate/up projection with the SwiGLU gating in the epilogue.  The plain
product is available too (tests and the microbenchmark compare it with the library's).
"""
from __future__ import annotations

import torch

from . import library as _library

_P, _I = _library._P, _library._I
_library.register_signatures({
    "dl_gemm_tc_bf16": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P],
})

MIN_ROWS = 17            # fewer rows go to the weight-streaming kernel
BLOCKS = 0               # > 0: persistent blocks (tuning and tests); 0: one per multiprocessor


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
                  _library.status_word(x.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    return out
