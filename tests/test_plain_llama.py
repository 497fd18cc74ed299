"""The plain implementation checked on its own: hand-computed cases in the manner of the
reference's kernel tests (tests/DotLLM.Tests.Unit/Cpu/Kernels/*.cs), invariants, and the llama3
frequency bands."""
import math

import numpy as np
import torch

import plain_llama as P
import tiny_models


def test_rms_norm_hand_calculated():
    out = P.rms_norm(torch.tensor([1.0, 2.0, 3.0, 4.0]), torch.tensor([1.0, 1.0, 2.0, 0.5]), 0.0)
    rms = math.sqrt(7.5)
    assert torch.allclose(out, torch.tensor([1 / rms, 2 / rms, 6 / rms, 2 / rms]), atol=1e-7)
    assert float(P.rms_norm(torch.zeros(4), torch.ones(4), 1e-5).abs().max()) == 0.0
    # eps sits inside the root, added to the mean
    x = torch.tensor([3.0, 4.0])
    assert torch.allclose(P.rms_norm(x, torch.ones(2), 0.5), x / math.sqrt(12.5 + 0.5))


def test_rope_hand_calculated_and_norm_preserving():
    cos, sin = P.rope_tables([0, 1, 2], 4, 10000.0)
    x = torch.tensor([[[1.0, 0.0, 0.0, 0.0]], [[1.0, 0.0, 0.0, 0.0]], [[0.0, 1.0, 0.0, 0.0]]])
    out = P.apply_rope(x, cos, sin)
    assert torch.allclose(out[0, 0], torch.tensor([1.0, 0.0, 0.0, 0.0]))                 # position 0: unchanged
    assert torch.allclose(out[1, 0], torch.tensor([math.cos(1), 0.0, math.sin(1), 0.0]), atol=1e-7)
    f1 = 10000.0 ** (-2 / 4)
    assert torch.allclose(out[2, 0], torch.tensor([0.0, math.cos(2 * f1), 0.0, math.sin(2 * f1)]), atol=1e-7)
    y = torch.randn(5, 3, 8, generator=torch.Generator().manual_seed(0))
    c, s = P.rope_tables(range(5), 8, 500000.0)
    assert torch.allclose(P.apply_rope(y, c, s).norm(dim=-1), y.norm(dim=-1), atol=1e-5)
    # partial rotation leaves the other dimensions alone (RoPETests.PartialRotation_OnlyFirstRopeDimRotated)
    c4, s4 = P.rope_tables(range(5), 4, 10000.0)
    assert torch.equal(P.apply_rope(y, c4, s4)[..., 4:], y[..., 4:])


def test_rope_dot_product_depends_on_distance_only():
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(1, 1, 16, generator=g), torch.randn(1, 1, 16, generator=g)
    def dot(pq, pk):
        cq, sq = P.rope_tables([pq], 16, 10000.0)
        ck, sk = P.rope_tables([pk], 16, 10000.0)
        return float((P.apply_rope(q, cq, sq) * P.apply_rope(k, ck, sk)).sum())
    assert abs(dot(10, 3) - dot(107, 100)) < 1e-4


def test_llama3_scaling_hits_all_three_bands():
    s = tiny_models.TINY_B["rope_scaling"]
    base = P.rope_frequencies(32, 500000.0)
    scaled = P.rope_frequencies(32, 500000.0, s)
    wavelen = 2 * math.pi / base
    keep = wavelen < 64 / 4.0
    divide = wavelen > 64 / 1.0
    blend = ~keep & ~divide
    assert keep.any() and divide.any() and blend.any()
    assert np.array_equal(scaled[keep], base[keep])
    assert np.allclose(scaled[divide], base[divide] / 8.0, rtol=1e-15)
    assert ((scaled[blend] < base[blend]) & (scaled[blend] > base[blend] / 8.0)).all()
    assert np.all(np.diff(scaled) < 0)                  # still decreasing
    assert np.array_equal(P.rope_frequencies(32, 500000.0, {"rope_type": "default"}), base)


def test_attention_causal_mask_gqa_and_window():
    g = torch.Generator().manual_seed(2)
    nh, nkv, hd, t = 4, 2, 8, 6
    q, k, v = torch.randn(t, nh * hd, generator=g), torch.randn(t, nkv * hd, generator=g), torch.randn(t, nkv * hd, generator=g)
    out = P.causal_attention(q, k, v, nh, nkv, 1 / math.sqrt(hd))
    # no future leakage: changing later keys and values leaves earlier outputs alone
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, -9.0
    out2 = P.causal_attention(q, k2, v2, nh, nkv, 1 / math.sqrt(hd))
    assert torch.equal(out[:4], out2[:4]) and not torch.allclose(out[4:], out2[4:])
    # the first token attends to itself only
    assert torch.allclose(out[0].view(nh, hd), v[0].view(nkv, hd).repeat_interleave(2, dim=0), atol=1e-6)
    # heads 0,1 read KV head 0 and heads 2,3 KV head 1 (AttentionTests.GQA_HeadBroadcast)
    q_same = q.clone()
    q_same[:, hd:2 * hd] = q_same[:, :hd]
    o = P.causal_attention(q_same, k, v, nh, nkv, 1 / math.sqrt(hd))
    assert torch.allclose(o[:, :hd], o[:, hd:2 * hd])
    # a chunk at an offset equals the tail of the whole (ApplyCausalMask_ChunkedPrefill_CorrectBoundary)
    tail = P.causal_attention(q[4:], k, v, nh, nkv, 1 / math.sqrt(hd), position_offset=4)
    assert torch.allclose(tail, out[4:], atol=1e-6)
    # window 2: query 5 sees keys 4 and 5 only
    w = P.causal_attention(q, k, v, nh, nkv, 1 / math.sqrt(hd), window=2)
    only = P.causal_attention(q[5:6], k[4:6], v[4:6], nh, nkv, 1 / math.sqrt(hd), position_offset=1)
    assert torch.allclose(w[5], only[0], atol=1e-6)
    # large scores stay finite (LargeScores_NumericallyStable)
    big = P.causal_attention(q * 1e3, k * 1e3, v, nh, nkv, 1.0)
    assert bool(torch.isfinite(big).all())


def test_swiglu_values():
    out = P.swiglu(torch.tensor([0.0, 1.0, -2.0]), torch.tensor([5.0, 2.0, 3.0]))
    want = torch.tensor([0.0, 2.0 / (1 + math.exp(-1.0)), -6.0 / (1 + math.exp(2.0))])
    assert torch.allclose(out, want, atol=1e-7)


def test_forward_prefix_property_and_determinism(tmp_path):
    folder = tiny_models.make_folder(tmp_path, "B")
    cfg, w = P.read_model_folder(folder)
    toks = tiny_models.random_tokens(80, cfg["vocab_size"], 3)
    full = P.forward(cfg, w, toks)
    assert full.shape == (80, cfg["vocab_size"]) and bool(torch.isfinite(full).all())
    assert torch.equal(full, P.forward(cfg, w, toks))
    assert torch.allclose(P.forward(cfg, w, toks[:33]), full[:33], atol=2e-6)     # causal: a prefix is a prefix
    # scaling matters beyond the original length only through the table: without it logits differ
    cfg2 = dict(cfg, rope_scaling=None)
    assert not torch.allclose(P.forward(cfg2, w, toks), full, atol=1e-3)
    a_cfg, a_w = P.read_model_folder(tiny_models.make_folder(tmp_path, "A"))
    assert "lm_head.weight" not in a_w and P.forward(a_cfg, a_w, [1, 2, 3]).shape == (3, 256)


def test_samplers():
    x = torch.tensor([1.0, 3.0, 3.0, 2.0, 3.0, -1.0])
    assert P.sample(x, [], temperature=0.0) == 1                                 # first maximum
    k2 = P.apply_top_k(x, 2)
    assert torch.isfinite(k2).tolist() == [False, True, True, False, False, False]   # ties in index order
    assert torch.equal(P.apply_top_k(x, 0), x) and torch.equal(P.apply_top_k(x, 6), x)
    probs = torch.tensor([0.5, 0.3, 0.15, 0.05])
    p = P.apply_top_p(torch.log(probs), 0.8)
    assert torch.isfinite(p).tolist() == [True, True, False, False]              # 0.5 + 0.3 reaches 0.8
    assert torch.isfinite(P.apply_top_p(torch.log(probs), 0.81)).tolist() == [True, True, True, False]
    m = P.apply_min_p(torch.log(probs), 0.25)
    assert torch.isfinite(m).tolist() == [True, True, True, False]               # 0.15/0.5 >= 0.25 > 0.05/0.5
    rp = P.apply_repetition_penalty(torch.tensor([2.0, -2.0, 1.0]), [0, 1, 0], 2.0, 0)
    assert rp.tolist() == [1.0, -4.0, 1.0]
    assert P.apply_repetition_penalty(torch.tensor([2.0, -2.0, 1.0]), [0, 1, 2], 2.0, 1).tolist() == [2.0, -2.0, 0.5]
    lg = torch.log(probs)
    assert [P.categorical(lg, r) for r in (0.0, 0.49, 0.51, 0.79, 0.81, 0.96)] == [0, 0, 1, 1, 2, 3]
    assert P.sample(lg, [], temperature=1.0, top_k=1, r=0.99) == 0


def test_parts_agree_with_the_reference_kernels_outputs():
    """kkokosa/dotLLM's own FP32 CUDA kernels (rmsnorm_f32, rope_f32 with the half-split pairing,
    attention_f32 at a position offset, swiglu_f32, add_f32, embedding_lookup_f32_f32out), compiled
    unmodified and run once on a B200: their outputs are committed in tests/golden/ with the script
    that made them.  The plain implementation's functions must reproduce them."""
    from golden import reference_kernels as rk
    golden = rk.load_golden()
    c = {k: golden[k] for k in rk.cases()}
    for name, value in rk.cases().items():                   # the inputs are the seeded ones of the script
        assert torch.equal(value, c[name]), name
    errs = rk.compare_with_plain(c, golden, P)
    for part, err in errs.items():
        assert err <= rk.BOUNDS[part], f"{part}: differs from the reference kernel's output by {err:.3e}"
