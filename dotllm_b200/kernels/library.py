"""Loads the compiled kernel library through ctypes and declares its entry points.

There is no fallback: if the library cannot be built or loaded, or the device is not
sm_100, every call raises ``KernelError``.
"""
from __future__ import annotations

import ctypes
import threading

from ..errors import KernelError

_P = ctypes.c_void_p
_I = ctypes.c_int
_F = ctypes.c_float

# name -> argument types (every function returns int status)
_SIGNATURES = {
    "dl_gather_rows": [_P, _I, _I, _P, _P, _I, _I, _I, _I, _P],
    "dl_add_rmsnorm": [_P, _P, _I, _P, _P, _I, _I, _I, _F, _P],
    "dl_rope_cache_write": [_P, _I, _P, _I, _P, _I, _I, _P, _P, _I, _I, _P, _P, _P, _I, _P, _P, _I,
                            _I, _I, _I, _I, _I, _P],
    "dl_attention_generic": [_P, _I, _P, _I, _I, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _F, _P, _P],
    "dl_swiglu": [_P, _P, _I, _P, _I, _I, _I, _P],
    "dl_gemm_f32": [_P, _I, _P, _P, _I, _I, _I, _I, _P],
    "dl_sample": [_P, _I, _I, _I, _P, _P, _P, _P, _P, _P, _I, _P],
    "dl_repetition_penalty": [_P, _I, _I, _I, _P, _I, _I, _P, _P, _P, _P, _P, _P, _P],
}

_lock = threading.Lock()
_lib = None
_checked_device = False


def declare(lib, signatures):
    for name, argtypes in signatures.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise KernelError(f"kernel library lacks entry point {name}") from exc
        fn.argtypes = argtypes
        fn.restype = ctypes.c_int


def library():
    """The loaded library (built on first use)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        from . import build
        path = build.build()
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as exc:
            raise KernelError(f"cannot load {path}: {exc}") from exc
        declare(lib, _SIGNATURES)
        lib.dl_last_error.restype = ctypes.c_char_p
        lib.dl_last_error.argtypes = []
        lib.dl_device_arch.restype = ctypes.c_int
        lib.dl_sm_count.restype = ctypes.c_int
        lib.dl_set_dependent_launch.restype = ctypes.c_int
        lib.dl_set_dependent_launch.argtypes = [ctypes.c_int]
        # Library products (cuBLAS through torch, used for bfloat16 prompts of more than 128 rows) must
        # accumulate and reduce in float32 like the kernels here: no bfloat16 split-k reductions.
        import torch
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        _lib = lib
        return lib


def register_signatures(signatures):
    """Entry points of kernels added later (each module declares its own)."""
    _SIGNATURES.update(signatures)
    if _lib is not None:
        declare(_lib, signatures)


def require_device():
    """Raise unless the current CUDA device can run the sm_100a kernels."""
    global _checked_device
    if _checked_device:
        return
    import torch
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: this library runs on NVIDIA B200 (sm_100) only "
                          "and has no CPU fallback")
    arch = library().dl_device_arch()
    if arch // 10 != 10:
        raise KernelError(f"the kernels are compiled for sm_100a; the current device reports "
                          f"compute capability {arch / 10:.1f}")
    _checked_device = True


def set_dependent_launch(on):
    """Switch programmatic dependent launch for later launches: kernels may begin, up to their
    first read of an earlier kernel's output, while that kernel is still finishing.  On unless
    the environment sets DOTLLM_DEPENDENT_LAUNCH=0; results are the same either way."""
    library().dl_set_dependent_launch(1 if on else 0)


_raw_stream = None


def current_stream():
    """The current CUDA stream's handle, for a kernel launch.  ``torch.cuda.current_stream()`` builds
    a Python stream object after several device-index and environment look-ups, 10 - 15 us a call with
    a few hundred launches a step; the handle alone comes from the binding underneath it."""
    global _raw_stream
    if _raw_stream is None:
        import torch
        raw, device = getattr(torch._C, "_cuda_getCurrentRawStream", None), getattr(torch._C, "_cuda_getDevice", None)
        if raw is not None and device is not None:
            _raw_stream = lambda: raw(device())
        else:
            _raw_stream = lambda: torch.cuda.current_stream().cuda_stream
    return _raw_stream()


def call(name, *args):
    lib = library()
    status = getattr(lib, name)(*args)
    if status != 0:
        raise KernelError(f"{name}: {lib.dl_last_error().decode(errors='replace')} (status {status})")


_status = {}
_counters = []
_STATUS_TEXT = {1: "a producer's wait for a free shared-memory stage expired",
                2: "a block table named a page outside the pool",
                3: "a consumer's wait for a bulk copy expired"}


def register_counters(tensor):
    """Arrival counters that kernels share between launches and leave zero.  A launch that gave up on
    a bounded wait may leave some of them counted; ``check_status`` clears them with the status word
    so that the launches after the error start from the state they expect."""
    _counters.append(tensor)


def status_word(device):
    """The per-device int32 that kernels with bounded waits set when a wait expires."""
    key = device.index
    if key not in _status:
        import torch
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def check_status():
    """Raise if a kernel reported an expired wait since the last check (synchronises)."""
    for key, word in _status.items():
        code = int(word.item())
        if code:
            word.zero_()
            for counters in _counters:
                if counters.device.index == key:
                    counters.zero_()
            raise KernelError(f"a kernel on cuda:{key} gave up: {_STATUS_TEXT.get(code, code)}")
