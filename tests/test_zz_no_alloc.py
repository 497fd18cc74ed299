"""The allocation-free product, called the way its users call it: through the exported C symbol,
with raw device pointers, from a place that has no allocator to offer.

Those users - a plug-in inside a host that froze its device memory at start-up, a control loop
that may not block on an allocator - hand over inputs and outputs they already own; the kernel's
scratch comes out of a fixed array inside the library.  The result must be what the ordinary
entry point gives, call after call, since every call reuses the same scratch.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbol():
    from dotllm_b200.kernels import build
    lib = ctypes.CDLL(str(build.build()))
    fn = lib.dl_gemm_skinny_bf16_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.dl_last_error.restype = ctypes.c_char_p
    lib.dl_gemm_skinny_static_status.restype = ctypes.c_int
    lib.dl_gemm_skinny_static_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    return lib, fn


def _static_status(lib, stream):
    code = ctypes.c_int(-1)
    assert lib.dl_gemm_skinny_static_status(ctypes.byref(code), stream) == 0, lib.dl_last_error().decode()
    return code.value


@pytest.mark.parametrize("M,N,K,fuse,out_dtype", [(8, 4096, 4096, 0, torch.float32), (3, 1000, 320, 0, torch.float32),
                                                  (16, 512, 2048, 1, torch.float32), (1, 6144, 512, 0, torch.float32),
                                                  (5, 1000, 320, 0, torch.bfloat16), (16, 512, 2048, 1, torch.bfloat16)])
def test_static_scratch_product_matches_the_ordinary_one(M, N, K, fuse, out_dtype, monkeypatch):
    from dotllm_b200.kernels import gemm_skinny
    monkeypatch.setattr(gemm_skinny, "SKINNY_ROWS", gemm_skinny.KERNEL_ROWS)      # the same kernel on both sides, up to its 16 rows
    lib, fn = _symbol()
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(40)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
    w = (torch.randn((2 if fuse else 1) * N, K, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    want = gemm_skinny.run(x, w, out_dtype, fuse_swiglu=bool(fuse))
    stream = torch.cuda.current_stream().cuda_stream
    code = 0 if out_dtype == torch.float32 else 1
    outs = [torch.full((M, N), float("nan"), dtype=out_dtype, device=dev) for _ in range(3)]
    # one warm-up call: the first call on a device looks up the array's address, and the first call
    # with a matrix encodes its tensor map
    assert fn(x.data_ptr(), K, w.data_ptr(), outs[2].data_ptr(), code, N, M, N, K, fuse, stream) == 0, lib.dl_last_error().decode()
    torch.cuda.synchronize()
    # Free device memory as the driver counts it: an allocation made behind torch's back (cudaMalloc,
    # cudaMallocAsync) inside the library would lower it; torch's own counter would not notice.
    free_before, _ = torch.cuda.mem_get_info(dev)
    torch_before = torch.cuda.memory_allocated(dev)
    for call in range(2):                                    # the second call finds the first one's leftovers
        status = fn(x.data_ptr(), K, w.data_ptr(), outs[call].data_ptr(), code, N, M, N, K, fuse, stream)
        assert status == 0, lib.dl_last_error().decode()
    assert _static_status(lib, stream) == 0                  # waits for the stream: no wait inside the kernels expired
    assert torch.cuda.mem_get_info(dev)[0] == free_before
    assert torch.cuda.memory_allocated(dev) == torch_before
    for call in range(2):
        out = outs[call]
        assert torch.allclose(out.float(), want.float(), rtol=2 ** -7, atol=2e-4), (call, float((out.float() - want.float()).abs().max()))
        assert torch.equal(out, want)                        # same arithmetic in the same order


def test_static_scratch_refuses_what_does_not_fit():
    lib, fn = _symbol()
    dev = torch.device("cuda", 0)
    M, N, K = 16, 16 * 20000, 64                             # more row tiles than the fixed scratch covers
    x = torch.zeros(M, K, dtype=torch.bfloat16, device=dev)
    w = torch.zeros(N, K, dtype=torch.bfloat16, device=dev)
    out = torch.zeros(M, N, dtype=torch.float32, device=dev)
    status = fn(x.data_ptr(), K, w.data_ptr(), out.data_ptr(), 0, N, M, N, K, 0,
                torch.cuda.current_stream().cuda_stream)
    assert status != 0 and b"built-in" in lib.dl_last_error()
