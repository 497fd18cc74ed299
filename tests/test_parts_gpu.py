"""Each part alone against the plain implementation, and a toy architecture defined here - a
mixer with state of its own, a windowed attention layer, a layer that runs twice, a layer that
reads another's cache, a feed-forward with routing - registered, built and stepped without
touching the package."""
from dataclasses import dataclass

import pytest
import torch

import plain_llama
import tiny_models
from dotllm_b200.kernels import ops

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def runtime(dtype=torch.float32):
    from dotllm_b200.parts import Runtime
    return Runtime(dtype, DEV)


def bind_random(part, seed, dtype):
    from dotllm_b200.weights import random_tensor
    tensors = {}
    for name, spec in part.weight_specs().items():
        t = random_tensor(name, spec, seed)
        tensors[name] = (t.to(dtype) if spec.role == "matrix" else t).to(DEV)
    part.bind(tensors)
    return {k: v.float().cpu() for k, v in tensors.items()}


def test_norm_part():
    from dotllm_b200.config import PartSpec
    from dotllm_b200.parts import make_part
    norm = make_part("norm", PartSpec("rmsnorm", {"eps": 1e-6, "gain_init": ("one_plus_uniform", 0.2)}), 200, runtime())
    w = bind_random(norm, 1, torch.float32)
    x = torch.randn(7, 200, generator=torch.Generator().manual_seed(0))
    d = torch.randn(7, 200, generator=torch.Generator().manual_seed(1))
    want = plain_llama.rms_norm(x, w["weight"], 1e-6)
    assert torch.allclose(norm.forward(x.to(DEV)).cpu(), want, atol=1e-5)
    res = x.to(DEV)
    got = norm.add_forward(res, d.to(DEV))
    assert torch.allclose(res.cpu(), x + d, atol=1e-6)
    assert torch.allclose(got.cpu(), plain_llama.rms_norm(x + d, w["weight"], 1e-6), atol=1e-5)


def test_rotary_part_tables_and_bands():
    from dotllm_b200.config import PartSpec
    from dotllm_b200.parts import make_part
    scaling = dict(tiny_models.TINY_B["rope_scaling"])
    pe = make_part("position_encoding", PartSpec("rotary", {"rotary_dim": 32, "head_dim": 32, "theta": 500000.0,
                                                            "max_positions": 256, "scaling": scaling}), 192, runtime())
    cos, sin = plain_llama.rope_tables(range(256), 32, 500000.0, scaling)
    assert torch.equal(pe.cos.cpu(), cos) and torch.equal(pe.sin.cpu(), sin)
    q = torch.randn(5, 3 * 32, generator=torch.Generator().manual_seed(2))
    pos = torch.tensor([0, 1, 63, 64, 255], dtype=torch.int32)
    d_q = q.to(DEV)
    pe.apply(d_q, None, pos.to(DEV))
    want = plain_llama.apply_rope(q.view(5, 3, 32), cos[pos.long()], sin[pos.long()]).reshape(5, 96)
    assert torch.allclose(d_q.cpu(), want, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from dotllm_b200.config import PartSpec
    from dotllm_b200.parts import make_part
    ffn = make_part("feed_forward", PartSpec("gated_mlp", {"intermediate_size": 176, "activation": "silu"}), 64,
                    runtime(dtype))
    w = bind_random(ffn, 3, dtype)
    weights = {"p.mlp." + k: v for k, v in w.items()}
    for rows in (3, 40):                                 # few rows: fused kernel; many: product + gating
        x = torch.randn(rows, 64, generator=torch.Generator().manual_seed(rows)).to(dtype)
        want = plain_llama.feed_forward_part(x.float(), weights, "p.")
        got = ops.resolve(ffn.forward(x.to(DEV))).float().cpu()     # few bfloat16 rows: the last product comes unlaunched
        assert torch.allclose(got, want, atol=1e-6 if dtype == torch.float32 else 2e-3)


def test_unlaunched_products_and_parts_that_do_not_fuse():
    """A part may return its last product unlaunched so that the next norm's addition and the next
    part's normalisation happen inside products.  A consumer that does not declare
    ``takes_scaled_rows``, and a norm that does not declare ``fuses_products``, must get plain tensors
    with the values of the separate kernels."""
    from dotllm_b200.config import PartSpec
    from dotllm_b200.parts import make_part
    from dotllm_b200.parts.base import Norm, normalised_for
    rt = runtime(torch.bfloat16)
    ffn = make_part("feed_forward", PartSpec("gated_mlp", {"intermediate_size": 176, "activation": "silu"}), 64, rt)
    bind_random(ffn, 3, torch.bfloat16)
    norm = make_part("norm", PartSpec("rmsnorm", {"eps": 1e-5, "gain_init": ("one_plus_uniform", 0.1)}), 64, rt)
    bind_random(norm, 4, torch.bfloat16)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(3, 64, generator=g).to(torch.bfloat16).to(DEV)
    stream0 = torch.randn(3, 64, generator=g).to(DEV)

    class PlainConsumer:
        pass

    class PlainNorm(Norm):
        def add_forward(self, residual, delta):
            assert isinstance(delta, torch.Tensor)
            residual += delta
            return residual.to(torch.bfloat16)

    pending = ffn.forward(x)
    assert isinstance(pending, ops.PendingProduct)
    want_stream = stream0.clone()
    want = norm.add_forward(want_stream, pending.tensor())
    # a consumer that fuses gets scaled rows standing for the same values
    s1 = stream0.clone()
    rows = normalised_for(ffn, norm, s1, ffn.forward(x))
    assert isinstance(rows, ops.ScaledRows) and torch.equal(s1, want_stream) and torch.equal(rows.tensor(), want)
    # a consumer that does not fuse gets the tensor
    s2 = stream0.clone()
    got = normalised_for(PlainConsumer(), norm, s2, ffn.forward(x))
    assert isinstance(got, torch.Tensor) and torch.equal(got, want) and torch.equal(s2, want_stream)
    # a norm that does not fuse gets a tensor to add
    s3 = stream0.clone()
    got = normalised_for(ffn, PlainNorm({}, 64, rt), s3, ffn.forward(x))
    assert isinstance(got, torch.Tensor) and torch.equal(s3, want_stream)


@pytest.mark.parametrize("rows", [40, 300])
def test_unlaunched_product_of_many_rows_adds_into_the_stream(rows):
    """Beyond the decode kernels' row counts an unlaunched product is the library's, with the stream as
    its accumulate operand: the stream and the normalised rows must equal a float64 product added in
    float32, and the values the separate way gives (product written, then added by the norm kernel)."""
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, 176, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(72, 176, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    gain = (1 + 0.1 * torch.randn(72, generator=g)).to(DEV)
    stream0 = torch.randn(rows, 72, generator=g).to(DEV)
    pending = ops.linear(x, w, out_dtype=torch.float32, resident=True, lazy=True)
    assert isinstance(pending, ops.PendingProduct)
    separate_stream = stream0.clone()
    separate = ops.add_rmsnorm(separate_stream, pending.tensor(), gain, 1e-5, torch.bfloat16)
    stream = stream0.clone()
    got = ops.add_rmsnorm(stream, pending, gain, 1e-5, torch.bfloat16, lazy=True)
    assert isinstance(got, torch.Tensor)
    want_stream = (stream0.double() + x.double() @ w.double().t()).float()
    assert torch.allclose(stream, want_stream, atol=2e-5, rtol=1e-5)
    assert torch.allclose(stream, separate_stream, atol=2e-6, rtol=1e-6)
    want = plain_llama.rms_norm(want_stream.cpu(), gain.cpu(), 1e-5)
    assert torch.allclose(got.float().cpu(), want, atol=2e-2, rtol=2e-2)
    assert torch.allclose(got.float(), separate.float(), atol=1e-2, rtol=1e-2)
    # a stream that is a view with gaps between its rows is not the library's operand: the separate way runs
    wide = torch.zeros(rows, 80, device=DEV)
    wide[:, :72] = stream0
    view = wide[:, :72]
    assert not pending.add_into(view) and torch.equal(view, stream0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts(dtype):
    from dotllm_b200.config import PartSpec
    from dotllm_b200.parts import make_part
    emb = make_part("embedding", PartSpec("token_embedding", {"vocab_size": 300}), 48, runtime(dtype))
    from types import SimpleNamespace
    head = make_part("head", PartSpec("linear_head", {"vocab_size": 300}), 48, runtime(dtype))
    w = bind_random(emb, 4, dtype)
    head.bind({"weight": emb.table})                              # a tied head is handed the embedding's table
    ids = torch.tensor([0, 299, 5, 5], dtype=torch.int32)
    h = emb.forward(SimpleNamespace(tokens=ids.to(DEV)))          # an embedding sees the step; this one reads its tokens
    assert h.dtype == torch.float32 and torch.equal(h.cpu(), w["weight"][ids.long()])
    logits = head.forward(h.to(dtype))
    want = w["weight"][ids.long()] @ w["weight"].T
    assert logits.dtype == torch.float32
    assert torch.allclose(logits.cpu(), want, atol=1e-6 if dtype == torch.float32 else 1e-4)


# ---------------------------------------------------------------------------------- a toy model
def toy_parts():
    """Parts defined in the test: a mixer with a decaying state per sequence, a position encoding
    that is not a rotation, and a feed-forward that routes each token to one of three experts."""
    from dotllm_b200.parts import (CacheNeed, FeedForward, Mixer, PositionEncoding, WeightSpec,
                                   register_feed_forward, register_mixer, register_position_encoding)

    class DecayMixer(Mixer):
        """s_t = a * s_{t-1} + x_t W_in ; y_t = s_t W_out.  Keeps s per sequence in the cache's
        fixed-size state."""

        def __init__(self, params, hidden_size, runtime):
            super().__init__(params, hidden_size, runtime)
            self.width = int(params["state_width"])
            self.decay = float(params["decay"])

        def weight_specs(self):
            return {"in_proj.weight": WeightSpec((self.width, self.hidden_size)),
                    "out_proj.weight": WeightSpec((self.hidden_size, self.width))}

        def bind(self, tensors):
            self.w_in, self.w_out = tensors["in_proj.weight"], tensors["out_proj.weight"]

        def cache_need(self):
            return CacheNeed("state", state_shape=(self.width,), state_dtype=torch.float32)

        def forward(self, x, step, view):
            u = x.float() @ self.w_in.float().T                      # [T, width]
            if step.attention_plan.all_single and not self.host_loop:
                # one token a sequence: all on the device, nothing read back (a step that a graph can hold)
                slots = view.slots.long()
                view.state[slots] = self.decay * view.state[slots] + u
                return (view.state[slots] @ self.w_out.float().T).to(torch.float32)
            out = torch.empty_like(u)
            seqs, slots = step.token_seq.tolist(), view.slots.tolist()
            for t in range(u.shape[0]):                              # tokens of a sequence arrive in order
                slot = slots[seqs[t]]
                view.state[slot] = self.decay * view.state[slot] + u[t]
                out[t] = view.state[slot]
            return (out @ self.w_out.float().T).to(torch.float32)

        host_loop = False

    class HostDecayMixer(DecayMixer):
        """The same mixer reading its indices on the host at every step, and saying so."""
        graph_safe = False
        host_loop = True

    class ShiftEncoding(PositionEncoding):
        """Adds pos * slope to the first dimension of every query and key head (not a rotation)."""

        def apply(self, q, k, positions):
            hd = int(self.params["head_dim"])
            shift = positions.float() * float(self.params["slope"])
            for x in (q, k):
                if x is not None:
                    x[:, ::hd] += shift[:, None].to(x.dtype)

    class RoutedFeedForward(FeedForward):
        """Top-1 routing in float32: expert e = argmax(x W_r^T); y = silu(x U_e^T) D_e^T."""

        def __init__(self, params, hidden_size, runtime):
            super().__init__(params, hidden_size, runtime)
            self.n_experts, self.inner = int(params["n_experts"]), int(params["inner"])

        def weight_specs(self):
            specs = {"router.weight": WeightSpec((self.n_experts, self.hidden_size), "precise", ("normal", 0.5))}
            for e in range(self.n_experts):
                specs[f"experts.{e}.up.weight"] = WeightSpec((self.inner, self.hidden_size))
                specs[f"experts.{e}.down.weight"] = WeightSpec((self.hidden_size, self.inner))
            return specs

        def bind(self, tensors):
            self.router = tensors["router.weight"]
            self.up = [tensors[f"experts.{e}.up.weight"] for e in range(self.n_experts)]
            self.down = [tensors[f"experts.{e}.down.weight"] for e in range(self.n_experts)]

        def forward(self, x):
            choice = (x.float() @ self.router.float().T).argmax(dim=1)
            out = torch.zeros(x.shape[0], self.hidden_size, dtype=torch.float32, device=x.device)
            for e in range(self.n_experts):                          # every expert on every row, the chosen one kept
                h = torch.nn.functional.silu(x.float() @ self.up[e].float().T)
                out += (choice == e)[:, None] * (h @ self.down[e].float().T)
            return out

    register_mixer("toy_decay", DecayMixer)
    register_mixer("toy_decay_host", HostDecayMixer)
    register_position_encoding("toy_shift", ShiftEncoding)
    register_feed_forward("toy_routed", RoutedFeedForward)


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int = 97
    hidden_size: int = 48
    architecture: str = "ToyForCausalLM"

    @classmethod
    def from_dict(cls, d):
        return cls(int(d["vocab_size"]), int(d["hidden_size"]), (d.get("architectures") or ["ToyForCausalLM"])[0])

    def to_dict(self):
        return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size}


def toy_spec(cfg, decay_mixer="toy_decay"):
    from dotllm_b200.config import ModelSpec, PartSpec, ScheduleEntry, pre_norm_layer
    norm = lambda p: PartSpec("rmsnorm", {"eps": 1e-5, "gain_init": ("one_plus_uniform", 0.1)}, p)
    ffn = lambda p, i: PartSpec("gated_mlp", {"intermediate_size": i, "activation": "silu"}, p)
    attn = PartSpec("attention", {"n_heads": 3, "n_kv_heads": 1, "head_dim": 16, "window": 40,
                                  "position": {"kind": "toy_shift", "params": {"head_dim": 16, "slope": 0.01}}},
                    "l0.attn.")
    decay = PartSpec(decay_mixer, {"state_width": 24, "decay": 0.9}, "l1.mix.")
    routed = PartSpec("toy_routed", {"n_experts": 3, "inner": 40}, "l1.moe.")
    layers = (pre_norm_layer(attn, ffn("l0.ffn.", 80), norm("l0.n1."), norm("l0.n2.")),
              pre_norm_layer(decay, routed, norm("l1.n1."), norm("l1.n2.")))
    # layer 0, layer 1, layer 1 again (its own state), layer 0 again reading the first run's cache
    schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1), ScheduleEntry(0, cache_of=0))
    return ModelSpec(cfg.architecture, cfg.hidden_size, cfg.vocab_size, 512,
                     PartSpec("token_embedding", {"vocab_size": cfg.vocab_size}, "emb."), layers, schedule,
                     norm("final."), PartSpec("linear_head", {"vocab_size": cfg.vocab_size}, "head."))


def toy_plain(w, tokens):
    """The toy model over a whole sequence with elementary operations."""
    n = len(tokens)
    h = w["emb.weight"][torch.tensor(tokens)]
    pos = torch.arange(n, dtype=torch.float32)
    kept = {}
    for e, (layer, share) in enumerate([(0, None), (1, None), (1, None), (0, 0)]):
        p = f"l{layer}."
        x = plain_llama.rms_norm(h, w[p + "n1.weight"], 1e-5)
        if layer == 0:
            q = (x @ w[p + "attn.q_proj.weight"].T).clone()
            q[:, ::16] += pos[:, None] * 0.01
            if share is None:
                k = (x @ w[p + "attn.k_proj.weight"].T).clone()
                k[:, ::16] += pos[:, None] * 0.01
                kept[e] = (k, x @ w[p + "attn.v_proj.weight"].T)
            k, v = kept[e if share is None else share]
            a = plain_llama.causal_attention(q, k, v, 3, 1, 0.25, window=40)
            h = h + a @ w[p + "attn.o_proj.weight"].T
        else:
            u = x @ w[p + "mix.in_proj.weight"].T
            s = torch.zeros(24)
            outs = []
            for t in range(n):
                s = 0.9 * s + u[t]
                outs.append(s.clone())
            h = h + torch.stack(outs) @ w[p + "mix.out_proj.weight"].T
        x = plain_llama.rms_norm(h, w[p + "n2.weight"], 1e-5)
        if layer == 0:
            g, u2 = x @ w[p + "ffn.gate_proj.weight"].T, x @ w[p + "ffn.up_proj.weight"].T
            h = h + plain_llama.swiglu(g, u2) @ w[p + "ffn.down_proj.weight"].T
        else:                                                        # each token goes to its best expert
            choice = (x @ w[p + "moe.router.weight"].T).argmax(dim=1).tolist()
            rows = []
            for t in range(n):
                up, down = w[p + f"moe.experts.{choice[t]}.up.weight"], w[p + f"moe.experts.{choice[t]}.down.weight"]
                hid = x[t] @ up.T
                rows.append((hid * torch.sigmoid(hid)) @ down.T)
            h = h + torch.stack(rows)
    return plain_llama.rms_norm(h, w["final.weight"], 1e-5) @ w["head.weight"].T


def test_toy_architecture_registers_builds_and_steps(tmp_path):
    from dotllm_b200 import Model, StepEntry
    from dotllm_b200.config import register_architecture
    from dotllm_b200.weights import write_random_model
    toy_parts()
    register_architecture("ToyForCausalLM", ToyConfig, toy_spec)
    folder = write_random_model(tmp_path / "toy", ToyConfig(), seed=2, dtype=torch.float32)
    _, w = plain_llama.read_model_folder(folder)
    model = Model.load(folder, dtype="float32")                     # the class is chosen by config.json
    assert model.spec.architecture == "ToyForCausalLM"
    cache = model.new_cache(64 * 6, max_sequences=3)
    kinds = sorted((g.kind, len(g.entries)) for g in cache.groups)
    assert kinds == [("kv", 1), ("state", 2)]                        # the shared execution owns no storage
    a = tiny_models.random_tokens(150, 97, 1)
    b = tiny_models.random_tokens(60, 97, 2)
    ra, rb = toy_plain(w, a), toy_plain(w, b)
    sa, sb = cache.open_sequence(), cache.open_sequence()
    got_a = [model.step(cache, [StepEntry(sa, a[:100], list(range(100))), StepEntry(sb, b[:7], [])])]
    got_b = []
    for t in range(100, 150):
        entries = [StepEntry(sa, [a[t]])]
        if t - 93 < 60:
            entries.append(StepEntry(sb, [b[t - 93]]))
        out = model.step(cache, entries)
        got_a.append(out[:1])
        if len(entries) == 2:
            got_b.append(out[1:2])
    assert float((torch.cat(got_a).cpu() - ra).abs().max()) < 5e-5
    assert float((torch.cat(got_b).cpu() - rb[7:57]).abs().max()) < 5e-5
    # the window released pages of the attention group; the state slot is zeroed for its next owner
    assert -1 in sa.pages[cache.kv_groups[0].index]
    slot = sb.slot
    cache.close_sequence(sb)
    sc = cache.open_sequence()
    assert sc.slot == slot
    out = model.step(cache, [StepEntry(sc, b[:30], list(range(30)))])
    assert float((out.cpu() - rb[:30]).abs().max()) < 5e-5
    cache.check()


def _toy_decode(model, w, step_fn, n_steps=14):
    """Three sequences of unequal lengths: prompts in one eager step, then ``n_steps`` decode steps
    through ``step_fn(cache, entries)``; every logit against the toy's plain form."""
    from dotllm_b200 import StepEntry
    cache = model.new_cache(64 * 8, max_sequences=4)
    starts = (20, 50, 3)
    reqs = [tiny_models.random_tokens(n + n_steps, 97, 40 + i) for i, n in enumerate(starts)]
    refs = [toy_plain(w, r) for r in reqs]
    seqs = [cache.open_sequence() for _ in reqs]
    out = model.step(cache, [StepEntry(s, r[:n]) for s, r, n in zip(seqs, reqs, starts)])
    for i, n in enumerate(starts):
        assert float((out[i].cpu() - refs[i][n - 1]).abs().max()) < 5e-5
    for t in range(n_steps):
        out = step_fn(cache, [StepEntry(s, [r[n + t]]) for s, r, n in zip(seqs, reqs, starts)])
        for i, n in enumerate(starts):
            assert float((out[i].cpu() - refs[i][n + t]).abs().max()) < 5e-5, f"step {t}, sequence {i}"
    cache.check()
    return cache


def test_toy_model_with_state_decodes_through_graphs(tmp_path, monkeypatch):
    """The toy model's decode steps as CUDA graphs: a graph per batch size, and graphs of a width with
    an idle row (three sequences in four rows: the idle row works on the cache's idle slot and page).
    The mixer's state must advance once in the step that captures (the trial run before the capture
    is undone).  A part that reads device values on the host says so (`graph_safe = False`) and the
    model then steps eagerly whatever the caller asks; a capture that fails although no part said so
    ends in a warning and eager steps."""
    from dotllm_b200 import Model
    from dotllm_b200.config import register_architecture
    from dotllm_b200.engine import decode_graph
    from dotllm_b200.weights import write_random_model
    toy_parts()
    register_architecture("ToyForCausalLM", ToyConfig, toy_spec)
    folder = write_random_model(tmp_path / "toy", ToyConfig(), seed=2, dtype=torch.float32)
    _, w = plain_llama.read_model_folder(folder)
    model = Model.load(folder, dtype="float32")
    assert model.decoder.graph_safe
    cache = _toy_decode(model, w, lambda cache, entries: model.step(cache, entries, graphs=True).clone())
    assert list(model.decode_graphs(cache).captured) == [3]
    cache = _toy_decode(model, w, lambda cache, entries: model.decode_graphs(cache).run(entries, capture_after=1).clone())
    assert list(model.decode_graphs(cache).captured) == [4]

    # the same model with a mixer that loops over its tokens on the host
    host_cfg = ToyConfig(architecture="ToyHostForCausalLM")
    register_architecture("ToyHostForCausalLM", ToyConfig, lambda cfg: toy_spec(cfg, "toy_decay_host"))
    host_folder = write_random_model(tmp_path / "toy_host", host_cfg, seed=2, dtype=torch.float32)
    _, hw = plain_llama.read_model_folder(host_folder)
    host_model = Model.load(host_folder, dtype="float32")
    assert not host_model.decoder.graph_safe
    cache = _toy_decode(host_model, hw, lambda cache, entries: host_model.step(cache, entries, graphs=True).clone())
    assert getattr(cache, "_decode_graphs", None) is None                 # nothing was captured

    # a capture that fails although every part claims to be safe: a warning, eager steps from then on
    def failing(decoder, ctx, cache):
        decoder.graph_safe = False
        raise decode_graph.CaptureFailed("a part waited for the device")
    monkeypatch.setattr(decode_graph, "capture_forward", failing)
    with pytest.warns(RuntimeWarning, match="waited for the device"):
        cache = _toy_decode(model, w, lambda cache, entries: model.step(cache, entries, graphs=True).clone())
    assert not model.decoder.graph_safe and not model.decode_graphs(cache).captured


# ------------------------------------------------------- a second toy: other shapes of layer and cache
def second_toy_parts():
    """Defined in the test, none of it in the package: a layer that is a mixer and nothing else (with
    two norms around it), an embedding that adds a learned position row, a mixer whose cache holds
    narrow latent keys and wide values in float32 whatever the run's type, and an attention mixer
    with capped scores and a penalty per head that grows with distance."""
    from dotllm_b200.kernels import ops
    from dotllm_b200.parts import (Arrangement, CacheNeed, Mixer, Part, WeightSpec, register_arrangement,
                                   register_embedding, register_mixer)

    class MixerOnly(Arrangement):
        """h = h + post(mixer(pre(h))): no feed-forward, a norm on either side of the mixer."""
        needs = ("pre", "mixer", "post")

        def forward(self, residual, pending, step, view):
            if pending is not None:
                residual += ops.resolve(pending).float()
            branch = self.mixer.forward(self.pre.forward(residual), step, view)
            return residual, self.post.forward(ops.resolve(branch).float().contiguous()).float()

    class PositionedEmbedding(Part):
        """h[t] = E[token[t]] + P[position[t]]: needs the step's positions, not only its tokens."""

        def weight_specs(self):
            return {"tokens.weight": WeightSpec((int(self.params["vocab_size"]), self.hidden_size)),
                    "positions.weight": WeightSpec((int(self.params["max_positions"]), self.hidden_size))}

        def bind(self, tensors):
            self.tokens, self.positions = tensors["tokens.weight"], tensors["positions.weight"]

        def forward(self, step):
            return ops.gather_rows(self.tokens, step.tokens) + ops.gather_rows(self.positions, step.token_pos)

    class LatentMixer(Mixer):
        """One head; keys are 8 numbers a token, values 24, kept in float32 pages.  Causal softmax
        attention over the latent keys, read and written by the mixer itself (plain tensor code)."""

        def weight_specs(self):
            h = self.hidden_size
            return {"q.weight": WeightSpec((8, h)), "k.weight": WeightSpec((8, h)), "v.weight": WeightSpec((24, h)),
                    "o.weight": WeightSpec((h, 24))}

        def bind(self, tensors):
            self.w = {k.split(".")[0]: v.float() for k, v in tensors.items()}

        def cache_need(self):
            return CacheNeed("kv", n_kv_heads=1, head_dim=8, k_dim=8, v_dim=24, dtype=torch.float32)

        def forward(self, x, step, view):
            assert view.k.dtype == torch.float32 and view.k.shape[1:] == (1, 64, 8) and view.v.shape[1:] == (1, 24, 64)
            xf = x.float()
            q, k, v = xf @ self.w["q"].T, xf @ self.w["k"].T, xf @ self.w["v"].T
            seqs, poss, table = step.token_seq.tolist(), step.token_pos.tolist(), view.block_table.tolist()
            out = torch.empty(x.shape[0], 24, device=x.device)
            for t, (b, pos) in enumerate(zip(seqs, poss)):
                view.k[table[b][pos // 64], 0, pos % 64] = k[t]
                view.v[table[b][pos // 64], 0, :, pos % 64] = v[t]
                keys = torch.stack([view.k[table[b][j // 64], 0, j % 64] for j in range(pos + 1)])
                vals = torch.stack([view.v[table[b][j // 64], 0, :, j % 64] for j in range(pos + 1)])
                out[t] = torch.softmax(keys @ q[t] * 0.5, dim=0) @ vals
            return out @ self.w["o"].T

    register_arrangement("toy_mixer_only", MixerOnly)
    register_embedding("toy_positioned", PositionedEmbedding)
    register_mixer("toy_latent", LatentMixer)


@dataclass(frozen=True)
class SecondToyConfig:
    vocab_size: int = 61
    hidden_size: int = 32
    architecture: str = "SecondToyForCausalLM"

    @classmethod
    def from_dict(cls, d):
        return cls(int(d["vocab_size"]), int(d["hidden_size"]))

    def to_dict(self):
        return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size}


SLOPES = (0.5, 0.05)


def second_toy_spec(cfg):
    from dotllm_b200.config import LayerPart, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, pre_norm_layer
    norm = lambda p: PartSpec("rmsnorm", {"eps": 1e-6, "gain_init": ("one_plus_uniform", 0.2)}, p)
    latent = LayerSpec("toy_mixer_only", (LayerPart("pre", "norm", norm("a.pre.")),
                                          LayerPart("mixer", "mixer", PartSpec("toy_latent", {}, "a.mix.")),
                                          LayerPart("post", "norm", norm("a.post."))))
    capped = pre_norm_layer(PartSpec("attention", {"n_heads": 2, "n_kv_heads": 2, "head_dim": 16, "window": None, "position": None,
                                                   "score": {"softcap": 3.0, "slopes": SLOPES}}, "b.attn."),
                            PartSpec("gated_mlp", {"intermediate_size": 56, "activation": "silu"}, "b.ffn."),
                            norm("b.n1."), norm("b.n2."))
    return ModelSpec("SecondToyForCausalLM", cfg.hidden_size, cfg.vocab_size, 200,
                     PartSpec("toy_positioned", {"vocab_size": cfg.vocab_size, "max_positions": 200}, "emb."),
                     (latent, capped), (ScheduleEntry(0), ScheduleEntry(1)), norm("final."),
                     PartSpec("linear_head", {"vocab_size": cfg.vocab_size}, "head."),
                     shared_weights=(("head.weight", "emb.tokens.weight"),))      # the head's matrix is the token table


def second_toy_plain(w, tokens):
    n = len(tokens)
    pos = torch.arange(n)
    h = w["emb.tokens.weight"][torch.tensor(tokens)] + w["emb.positions.weight"][pos]
    x = plain_llama.rms_norm(h, w["a.pre.weight"], 1e-6)
    q, k, v = x @ w["a.mix.q.weight"].T, x @ w["a.mix.k.weight"].T, x @ w["a.mix.v.weight"].T
    s = (q @ k.T) * 0.5
    s = s.masked_fill(pos[None, :] > pos[:, None], float("-inf"))
    h = h + plain_llama.rms_norm(torch.softmax(s, dim=1) @ v @ w["a.mix.o.weight"].T, w["a.post.weight"], 1e-6)
    x = plain_llama.rms_norm(h, w["b.n1.weight"], 1e-6)
    q, k, v = (x @ w[f"b.attn.{n_}_proj.weight"].T for n_ in "qkv")
    heads = []
    for hd in range(2):
        sl = slice(16 * hd, 16 * hd + 16)
        s = (q[:, sl] @ k[:, sl].T) * 0.25
        s = 3.0 * torch.tanh(s / 3.0) + SLOPES[hd] * (pos[None, :] - pos[:, None]).float()
        s = s.masked_fill(pos[None, :] > pos[:, None], float("-inf"))
        heads.append(torch.softmax(s, dim=1) @ v[:, sl])
    h = h + torch.cat(heads, dim=1) @ w["b.attn.o_proj.weight"].T
    x = plain_llama.rms_norm(h, w["b.n2.weight"], 1e-6)
    h = h + plain_llama.swiglu(x @ w["b.ffn.gate_proj.weight"].T, x @ w["b.ffn.up_proj.weight"].T) @ w["b.ffn.down_proj.weight"].T
    return plain_llama.rms_norm(h, w["final.weight"], 1e-6) @ w["emb.tokens.weight"].T


def test_second_toy_other_layer_shapes_cache_widths_and_score_hook(tmp_path):
    """A mixer-only layer with norms of its own names, an embedding that reads positions, a cache
    group with narrow keys, wide values and its own storage type, scores capped and biased before
    the softmax, and a head that shares the embedding's matrix through the description: all of it
    registered, built, loaded and stepped (prompt, then token by token, two sequences) without a
    change to the package, and equal to plain code."""
    from dotllm_b200 import Model, StepEntry
    from dotllm_b200.config import register_architecture
    from dotllm_b200.weights import write_random_model
    second_toy_parts()
    register_architecture("SecondToyForCausalLM", SecondToyConfig, second_toy_spec)
    folder = write_random_model(tmp_path / "toy2", SecondToyConfig(), seed=4, dtype=torch.float32)
    _, w = plain_llama.read_model_folder(folder)
    assert "head.weight" not in w                                       # a shared tensor is stored once
    for dtype, bound in (("float32", 5e-5), ("bfloat16", 6e-2)):
        model = Model.load(folder, dtype=dtype)
        assert model.decoder.head.weight is model.decoder.embedding.tokens
        cache = model.new_cache(64 * 8, max_sequences=2)
        latent = [g for g in cache.kv_groups if g.k.shape[-1] == 8][0]
        assert latent.k.dtype == torch.float32 and latent.v.shape[-2] == 24 and latent.bytes_per_token() == 4 * 32
        a, b = tiny_models.random_tokens(90, 61, 11), tiny_models.random_tokens(70, 61, 12)
        ra, rb = second_toy_plain(w, a), second_toy_plain(w, b)
        sa, sb = cache.open_sequence(), cache.open_sequence()
        got_a = [model.step(cache, [StepEntry(sa, a[:70], list(range(70))), StepEntry(sb, b[:50], [49])])[:70]]
        got_b = []
        for t in range(20):
            out = model.step(cache, [StepEntry(sb, [b[50 + t]]), StepEntry(sa, [a[70 + t]])])
            got_b.append(out[:1])
            got_a.append(out[1:2])
        assert float((torch.cat(got_a).cpu() - ra).abs().max()) < bound
        assert float((torch.cat(got_b).cpu() - rb[50:70]).abs().max()) < bound
        cache.close_sequence(sa)
        cache.close_sequence(sb)
        cache.check()


def test_random_model_in_memory_equals_the_folder_it_would_write(tmp_path):
    """Model.random(config, seed) and write_random_model(config, seed) loaded back are the same model."""
    from dotllm_b200 import Model
    from dotllm_b200.config import config_from_dict
    from dotllm_b200.weights import write_random_model
    cfg = config_from_dict(tiny_models.TINY_B)
    for dtype in (torch.bfloat16, torch.float32):
        folder = write_random_model(tmp_path / f"b_{dtype}", cfg, seed=9, dtype=dtype)
        loaded, made = Model.load(folder, dtype=dtype), Model.random(cfg, seed=9, dtype=dtype)
        for (_, p), (_, q) in zip(loaded.decoder.named_parts(), made.decoder.named_parts()):
            for name, value in vars(p).items():
                if isinstance(value, torch.Tensor):
                    assert torch.equal(value, getattr(q, name)), name
