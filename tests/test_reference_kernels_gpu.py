"""The plain implementation against kkokosa/dotLLM's own FP32 CUDA kernels, compiled unmodified at
test time (see tests/golden/reference_kernels.py).  Skipped where the reference's kernel sources
are not at hand."""
import pytest

import plain_llama
from golden import reference_kernels as rk

pytestmark = pytest.mark.gpu


def test_plain_parts_agree_with_the_reference_kernels():
    if rk.kernel_sources() is None:
        pytest.skip("the reference's native/kernels/*.cu are not available on this machine")
    lib = rk.build()
    c = rk.cases()
    ref = rk.run(lib, c)
    errs = rk.compare_with_plain(c, ref, plain_llama)
    for part, err in errs.items():
        assert err <= rk.BOUNDS[part], f"{part}: plain implementation and reference kernel differ by {err:.3e}"
    # and the committed outputs are those of the kernels as they are now
    golden = rk.load_golden()
    for name, value in ref.items():
        assert float((golden[name] - value).abs().max()) <= 1e-6, name


def test_the_product_kernels_agree_with_the_reference_kernels():
    """The package's own float32 kernels on the same inputs: norm and gating."""
    if rk.kernel_sources() is None:
        pytest.skip("the reference's native/kernels/*.cu are not available on this machine")
    import torch
    from dotllm_b200.kernels import ops
    c = rk.cases()
    ref = rk.run(rk.build(), c)
    x = c["norm_x"].cuda()
    y = ops.add_rmsnorm(x.clone(), None, c["norm_w"].cuda(), float(c["norm_eps"]), torch.float32)
    assert float((y.cpu() - ref["norm_y"]).abs().max()) <= 2e-5
    s = ops.swiglu(torch.cat([c["gate"], c["up"]], dim=1).cuda().contiguous())
    assert float((s.cpu() - ref["swiglu_out"]).abs().max()) <= 2e-6
