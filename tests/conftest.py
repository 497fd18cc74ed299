import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (NVIDIA B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def cpu_kernels(monkeypatch):
    """Replace the CUDA kernel wrappers by their plain torch references so that the engine's
    host logic (step planning, cache addressing, block wiring) can run without a GPU."""
    import kernel_refs
    from dotllm_b200.kernels import ops
    for name in ("gather_rows", "add_rmsnorm", "rope_cache_write", "attention", "swiglu", "linear", "gated_linear",
                 "sample", "repetition_penalty"):
        monkeypatch.setattr(ops, name, getattr(kernel_refs, name))
    # ops.rope_cache_attention composes the two patched functions above for anything but CUDA bfloat16
    return kernel_refs
