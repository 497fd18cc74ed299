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


def pytest_terminal_summary(terminalreporter):
    """The worst logit errors the parity tests saw, next to the bounds they were held to."""
    try:
        import engine_checks
    except ImportError:
        return
    for dtype, (rel_max, rel_rms, abs_max) in engine_checks.OBSERVED.items():
        terminalreporter.write_line(f"observed {dtype}: max |diff| {abs_max:.3e}, max |diff| / row rms {rel_max:.3e}, "
                                    f"row rms error / row rms {rel_rms:.3e}")
