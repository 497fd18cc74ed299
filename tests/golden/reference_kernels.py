"""kkokosa/dotLLM's own FP32 CUDA kernels, compiled unmodified and run on small inputs.

The reference's model code is C# and cannot be compiled or imported here, but its FP32 kernels for
every part that is not a matrix product are plain CUDA C (native/kernels/rmsnorm_f32.cu, rope_f32.cu
with rope_type = 1 for the half-split pairing, attention_f32.cu, swiglu_f32.cu, add_f32.cu,
embedding_f32out.cu; launch shapes as in src/DotLLM.Cuda/CudaKernels.cs:197-348).  This module
`#include`s those files, as they are, into a launcher of a few lines, compiles it with nvcc into the
git-ignored ``baseline/_ref/`` and runs the kernels on a GPU.  Nothing of it enters the package.

    python tests/golden/reference_kernels.py        # on a GPU box: rewrites reference_kernels.npz

``reference_kernels.npz`` (committed beside this file) holds the inputs and the kernels' outputs of
``cases()``; tests/test_plain_llama.py compares the plain implementation with them on the CPU, and
tests/test_reference_kernels_gpu.py reruns the kernels when their sources are at hand.
The sources are looked for in the reference checkout and in ``baseline/_ref/native_kernels`` (where
``__graft_entry__.build()`` copies them so that they travel to a machine without the checkout).
"""
from __future__ import annotations

import ctypes
import math
import os
import shutil
import subprocess
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
REF_DIR = ROOT / "baseline" / "_ref"
KERNEL_FILES = ("rmsnorm_f32.cu", "rope_f32.cu", "attention_f32.cu", "swiglu_f32.cu", "add_f32.cu", "embedding_f32out.cu")
GOLDEN = Path(__file__).with_name("reference_kernels.npz")

LAUNCHER = r'''
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
%(includes)s
// Launch shapes of src/DotLLM.Cuda/CudaKernels.cs:197-348: one block of 256 threads per row (norm,
// embedding, attention: per query token and head), 256-thread blocks over elements otherwise;
// attention's shared memory is (head_dim + 256 + head_dim + 32) floats.
extern "C" int ref_rmsnorm(const float* x, const float* w, float* y, int rows, int n, float eps) {
    rmsnorm_f32<<<rows, 256>>>(x, w, y, n, eps);
    return (int)cudaDeviceSynchronize();
}
extern "C" int ref_rope(float* q, float* k, const int* pos, int T, int nh, int nkv, int hd, int rope_dim, float theta, int type) {
    const int pairs = T * (nh > nkv ? nh : nkv) * (rope_dim / 2);
    rope_f32<<<(pairs + 255) / 256, 256>>>(q, k, pos, T, nh, nkv, hd, rope_dim, theta, type);
    return (int)cudaDeviceSynchronize();
}
extern "C" int ref_attention(const float* q, const float* k, const float* v, float* out, int seq_q, int seq_kv, int nh, int nkv,
                             int hd, int position_offset, int window) {
    const size_t smem = (size_t)(hd + 256 + hd + 32) * sizeof(float);
    attention_f32<<<seq_q * nh, 256, smem>>>(q, k, v, out, seq_q, seq_kv, nh, nkv, hd, position_offset, window);
    return (int)cudaDeviceSynchronize();
}
extern "C" int ref_swiglu(const float* g, const float* u, float* out, int n, int T) {
    swiglu_f32<<<(n * T + 255) / 256, 256>>>(g, u, out, n, T);
    return (int)cudaDeviceSynchronize();
}
extern "C" int ref_add(const float* a, const float* b, float* out, int n) {
    add_f32<<<(n + 255) / 256, 256>>>(a, b, out, n);
    return (int)cudaDeviceSynchronize();
}
extern "C" int ref_embedding(const float* table, const int* ids, float* out, int T, int hidden) {
    embedding_lookup_f32_f32out<<<T, 256>>>(table, ids, out, T, hidden);
    return (int)cudaDeviceSynchronize();
}
'''


def reference_checkout():
    """The reference's source tree: $DOTLLM_REFERENCE_ROOT, or a folder `reference` beside the repository."""
    root = os.environ.get("DOTLLM_REFERENCE_ROOT")
    return Path(root) if root else Path(__file__).resolve().parents[3] / "reference"


def kernel_sources():
    """Folder with the reference's kernel files, or None."""
    for cand in (reference_checkout() / "native" / "kernels", REF_DIR / "native_kernels"):
        if all((cand / f).is_file() for f in KERNEL_FILES):
            return cand
    return None


def stage_sources():
    """Copy the kernel files (unchanged) into baseline/_ref/native_kernels so that they travel with
    the working tree to a machine that has no reference checkout.  True if they are there."""
    src = reference_checkout() / "native" / "kernels"
    dst = REF_DIR / "native_kernels"
    if all((src / f).is_file() for f in KERNEL_FILES):
        dst.mkdir(parents=True, exist_ok=True)
        for f in KERNEL_FILES:
            shutil.copyfile(src / f, dst / f)
    return all((dst / f).is_file() for f in KERNEL_FILES)


def build():
    """Compile the launcher around the unmodified kernel files; returns the loaded library."""
    src = kernel_sources()
    if src is None:
        raise FileNotFoundError("the reference's native/kernels/*.cu are not available")
    REF_DIR.mkdir(parents=True, exist_ok=True)
    cu, so = REF_DIR / "ref_launch.cu", REF_DIR / "libref_kernels.so"
    cu.write_text(LAUNCHER % {"includes": "\n".join(f'#include "{src / f}"' for f in KERNEL_FILES)})
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    res = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-shared", "-Xcompiler", "-fPIC",
                          "-o", str(so), str(cu)], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on the reference kernels:\n{res.stdout}\n{res.stderr}")
    return ctypes.CDLL(str(so))


def cases(seed=5):
    """Small inputs (CPU tensors): sizes off every power of two, GQA 3:1, a prompt continued at an
    offset (the chunked-prefill mask), rows of very different scale for the norm."""
    g = torch.Generator().manual_seed(seed)
    r = lambda *shape: torch.randn(*shape, generator=g)
    T, nh, nkv, hd = 13, 6, 2, 48
    c = {
        "norm_x": r(5, 200) * torch.tensor([0.01, 1.0, 30.0, 1.0, 5.0])[:, None], "norm_w": 1 + 0.2 * r(200), "norm_eps": torch.tensor(1e-5),
        "rope_q": r(T, nh * hd), "rope_k": r(T, nkv * hd), "rope_pos": torch.arange(7, 7 + T, dtype=torch.int32),
        "rope_theta": torch.tensor(10000.0), "rope_dim": torch.tensor(hd),
        "attn_q": r(5, nh * hd), "attn_k": r(21, nkv * hd), "attn_v": r(21, nkv * hd), "attn_offset": torch.tensor(16),
        "gate": r(7, 176) * 3, "up": r(7, 176),
        "add_a": r(333), "add_b": r(333),
        "embed_table": r(50, 72), "embed_ids": torch.tensor([3, 49, 0, 3, 17], dtype=torch.int32),
    }
    c["shape"] = torch.tensor([T, nh, nkv, hd])
    return c


def run(lib, c, device="cuda"):
    """The reference kernels' outputs for ``cases()``, as CPU tensors."""
    d = {k: v.to(device) for k, v in c.items() if v.dim() > 0 and k != "shape"}
    T, nh, nkv, hd = (int(v) for v in c["shape"])
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    out = {}
    y = torch.empty_like(d["norm_x"])
    assert lib.ref_rmsnorm(p(d["norm_x"]), p(d["norm_w"]), p(y), y.shape[0], y.shape[1], ctypes.c_float(float(c["norm_eps"]))) == 0
    out["norm_y"] = y
    q, k = d["rope_q"].clone(), d["rope_k"].clone()
    assert lib.ref_rope(p(q), p(k), p(d["rope_pos"]), T, nh, nkv, hd, int(c["rope_dim"]), ctypes.c_float(float(c["rope_theta"])), 1) == 0
    out["rope_q_out"], out["rope_k_out"] = q, k
    o = torch.empty_like(d["attn_q"])
    assert lib.ref_attention(p(d["attn_q"]), p(d["attn_k"]), p(d["attn_v"]), p(o), o.shape[0], d["attn_k"].shape[0], nh, nkv, hd,
                             int(c["attn_offset"]), 0) == 0
    out["attn_out"] = o
    s = torch.empty_like(d["gate"])
    assert lib.ref_swiglu(p(d["gate"]), p(d["up"]), p(s), s.shape[1], s.shape[0]) == 0
    out["swiglu_out"] = s
    a = torch.empty_like(d["add_a"])
    assert lib.ref_add(p(d["add_a"]), p(d["add_b"]), p(a), a.numel()) == 0
    out["add_out"] = a
    e = torch.empty(d["embed_ids"].numel(), d["embed_table"].shape[1], device=device)
    assert lib.ref_embedding(p(d["embed_table"]), p(d["embed_ids"]), p(e), e.shape[0], e.shape[1]) == 0
    out["embed_out"] = e
    return {k: v.cpu() for k, v in out.items()}


def compare_with_plain(c, ref, plain):
    """Largest |plain implementation - reference kernel| per part (``plain`` is tests/plain_llama)."""
    T, nh, nkv, hd = (int(v) for v in c["shape"])
    err = lambda a, b: float((a - b).abs().max())
    cos, sin = plain.rope_tables(c["rope_pos"].tolist(), int(c["rope_dim"]), float(c["rope_theta"]))
    return {
        "rms_norm": err(plain.rms_norm(c["norm_x"], c["norm_w"], float(c["norm_eps"])), ref["norm_y"]),
        "rope_q": err(plain.apply_rope(c["rope_q"].view(T, nh, hd), cos, sin).reshape(T, -1), ref["rope_q_out"]),
        "rope_k": err(plain.apply_rope(c["rope_k"].view(T, nkv, hd), cos, sin).reshape(T, -1), ref["rope_k_out"]),
        "attention": err(plain.causal_attention(c["attn_q"], c["attn_k"], c["attn_v"], nh, nkv, 1.0 / math.sqrt(hd),
                                                position_offset=int(c["attn_offset"])), ref["attn_out"]),
        "swiglu": err(plain.swiglu(c["gate"], c["up"]), ref["swiglu_out"]),
        "add": err(c["add_a"] + c["add_b"], ref["add_out"]),
        "embedding": err(plain.embed(c["embed_table"], c["embed_ids"].tolist()), ref["embed_out"]),
    }


# What the two may differ by: float32 summation order and the device's expf; the kernel computes rope
# angles in float32 (powf, cosf of up to 20 rad) where the plain implementation rounds float64 tables;
# gated values reach about 30.
BOUNDS = {"rms_norm": 2e-5, "rope_q": 2e-5, "rope_k": 2e-5, "attention": 2e-6, "swiglu": 4e-6, "add": 0.0, "embedding": 0.0}


def load_golden():
    data = np.load(GOLDEN)
    return {k: torch.from_numpy(data[k]) for k in data.files}


if __name__ == "__main__":
    import sys
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    import plain_llama
    c = cases()
    ref = run(build(), c)
    np.savez_compressed(GOLDEN, **{k: v.numpy() for k, v in {**c, **ref}.items()})
    print({k: f"{v:.2e}" for k, v in compare_with_plain(c, ref, plain_llama).items()})
    print(f"wrote {GOLDEN} ({os.path.getsize(GOLDEN)} bytes)")
