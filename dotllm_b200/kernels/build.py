"""Compiles the CUDA sources under ``csrc/`` for sm_100a into one shared library.

The library is built in-tree (``csrc/_build/``) the first time it is needed and again
whenever a source, a header or the flags change.  Only ``nvcc`` is needed: the sources
include no PyTorch headers and the library is loaded through ``ctypes``.  If the tree is
not writable the build goes to a per-user folder under the system's temporary directory.
Progress goes to standard error, one line per file, so that a first call that compiles
for a minute is seen to be alive.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor, as_completed
from pathlib import Path

from ..errors import KernelError

CSRC = Path(__file__).resolve().parent.parent / "csrc"
LIB_NAME = "libdotllm_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# --use_fast_math is left off on purpose: softmax, norms and sampling use exact expf/sqrtf.
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=default"]
# Extra compiler flags for debugging builds, e.g. DOTLLM_NVCC_EXTRA="-DDL_SELF_CHECK=1" makes the
# kernels that support it verify their own shared-memory addresses and record a status code
# instead of touching memory outside their buffers.
NVCC_FLAGS += os.environ.get("DOTLLM_NVCC_EXTRA", "").split()


def _log(msg):
    print(f"[dotllm_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelError("nvcc not found: the CUDA kernels cannot be compiled "
                      "(set NVCC or CUDA_HOME, or put nvcc on PATH)")


def sources():
    return sorted(CSRC.glob("*.cu"))


def _headers():
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))


def _digest(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in paths:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _writable_dir(path):
    try:
        path.mkdir(parents=True, exist_ok=True)
        probe = path / f".probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir():
    in_tree = CSRC / "_build"
    if _writable_dir(in_tree):
        return in_tree
    tag = hashlib.sha256(str(CSRC).encode()).hexdigest()[:12]
    fallback = Path(tempfile.gettempdir()) / f"dotllm_b200_build_{os.getuid()}_{tag}"
    if _writable_dir(fallback):
        return fallback
    raise KernelError(f"neither {in_tree} nor {fallback} is writable: nowhere to build the kernels")


def _up_to_date(out_dir):
    """The library path if a library built from the present sources exists in ``out_dir``."""
    manifest = out_dir / "manifest.json"
    lib = out_dir / LIB_NAME
    if not (manifest.is_file() and lib.is_file()):
        return None
    try:
        recorded = json.loads(manifest.read_text())
    except (OSError, json.JSONDecodeError):
        return None
    header_digest = _digest(_headers(), " ".join(ARCH_FLAGS + NVCC_FLAGS))
    wanted = {src.name: _digest([src], header_digest) for src in sources()}
    return lib if recorded.get("objects") == wanted else None


def existing_library():
    """A current library from the tree or the fallback folder, without building."""
    in_tree = CSRC / "_build"
    if in_tree.is_dir():
        lib = _up_to_date(in_tree)
        if lib:
            return lib
    return None


def build(verbose=True, ptxas_info=False):
    """Compile what changed and link.  Returns the path of the shared library."""
    lib = existing_library()
    if lib:
        return lib
    out_dir = build_dir()
    lib = _up_to_date(out_dir)
    if lib:
        return lib
    nvcc = find_nvcc()
    import fcntl
    with open(out_dir / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        lib = _up_to_date(out_dir)              # another process may have built it meanwhile
        if lib:
            return lib
        header_digest = _digest(_headers(), " ".join(ARCH_FLAGS + NVCC_FLAGS))
        try:
            recorded = json.loads((out_dir / "manifest.json").read_text()).get("objects", {})
        except (OSError, json.JSONDecodeError):
            recorded = {}
        srcs = sources()
        wanted = {src.name: _digest([src], header_digest) for src in srcs}
        todo = [s for s in srcs
                if recorded.get(s.name) != wanted[s.name] or not (out_dir / (s.stem + ".o")).is_file()]
        if verbose:
            _log(f"compiling {len(todo)} of {len(srcs)} CUDA sources for sm_100a into {out_dir}")
        t0 = time.time()

        def compile_one(src):
            cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src),
                   "-o", str(out_dir / (src.stem + ".o"))]
            if ptxas_info:
                cmd.insert(1, "-Xptxas=-v")
            res = subprocess.run(cmd, capture_output=True, text=True)
            return src, res

        done = 0
        with ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as pool:
            futures = [pool.submit(compile_one, s) for s in todo]
            for fut in as_completed(futures):
                src, res = fut.result()
                done += 1
                if res.returncode != 0:
                    raise KernelError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
                if verbose:
                    _log(f"  [{done}/{len(todo)}] {src.name} ({time.time() - t0:.0f} s)")
                if ptxas_info and res.stderr:
                    sys.stderr.write(res.stderr)
        link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(out_dir / (LIB_NAME + ".tmp")),
                *[str(out_dir / (s.stem + ".o")) for s in srcs]]
        res = subprocess.run(link, capture_output=True, text=True)
        if res.returncode != 0:
            raise KernelError(f"linking {LIB_NAME} failed:\n{res.stdout}\n{res.stderr}")
        os.replace(out_dir / (LIB_NAME + ".tmp"), out_dir / LIB_NAME)
        (out_dir / "manifest.json").write_text(json.dumps({"objects": wanted}, indent=1))
        if verbose:
            _log(f"built {LIB_NAME} in {time.time() - t0:.0f} s")
        return out_dir / LIB_NAME


if __name__ == "__main__":
    print(build(ptxas_info="-v" in sys.argv))
