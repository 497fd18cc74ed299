"""The engine against the plain implementation, in float32 and bfloat16, under every cut:
whole requests, the last 32 tokens one by one, unequal batches with early finishers and reused
slots, long decoding, the first tokens, and greedy generation through the entry point."""
import pytest
import torch

import plain_llama
import tiny_models
from engine_checks import TOL, assert_close, first_wrong, greedy_ok, load_pair

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def requests_for(which, cfg):
    lens = {"A": [5, 11, 17, 100, 64, 65, 128], "B": [1, 9, 33, 70, 200, 256, 63],
            "C": [300, 40, 129, 7, 1000], "D": [260, 33, 129, 1, 700]}[which]
    return [tiny_models.random_tokens(n, cfg["vocab_size"], seed=100 + i) for i, n in enumerate(lens)]


@pytest.fixture(scope="module")
def tmp(tmp_path_factory):
    return tmp_path_factory.mktemp("models")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
def test_whole_tail_and_batched(tmp, which, dtype):
    from dotllm_b200 import StepEntry
    model, cfg, weights, _ = load_pair(tmp, which, dtype)
    reqs = requests_for(which, cfg)
    refs = [plain_llama.forward(cfg, weights, r) for r in reqs]
    longest = max(len(r) for r in reqs)
    cache = model.new_cache(max_tokens=2 * ((longest + 63) // 64 * 64) + 128)

    # 1. each request alone and whole, every position wanted
    for i, (r, ref) in enumerate(zip(reqs, refs)):
        cache.fill_free_pages(float("nan"))
        s = cache.open_sequence()
        out = model.step(cache, [StepEntry(s, r, list(range(len(r))))])
        cache.close_sequence(s)
        assert first_wrong(out, ref, dtype) is None, \
            f"whole: request {i} first wrong position {first_wrong(out, ref, dtype)}"

    # 2. the last 32 tokens one by one (shorter requests: everything one by one)
    for i, (r, ref) in enumerate(zip(reqs, refs)):
        cache.fill_free_pages(float("nan"))
        s = cache.open_sequence()
        head = max(0, len(r) - 32)
        got = []
        if head:
            got.append(model.step(cache, [StepEntry(s, r[:head], list(range(head)))]))
        for t in range(head, len(r)):
            got.append(model.step(cache, [StepEntry(s, [r[t]])]))
        cache.close_sequence(s)
        out = torch.cat(got)
        assert first_wrong(out, ref, dtype) is None, \
            f"tail: request {i} (head {head}) first wrong position {first_wrong(out, ref, dtype)}"
    cache.check()

    # 3. unequal batches: prompts whole in one step (all but the last k_b tokens), then one token
    # each; shorter requests end earlier; batches follow one another and reuse slots and pages.
    # The cache is sized for one batch only.
    batches = [reqs[:3], reqs[3:5], reqs[5:]]
    need = max(sum((len(r) + 63) // 64 * 64 for r in b) for b in batches if b)
    small = model.new_cache(max_tokens=need)
    for bi, batch in enumerate(batches):
        if not batch:
            continue
        small.fill_free_pages(float("nan"))
        seqs = [small.open_sequence() for _ in batch]
        tails = [min(len(r) - 1, 3 + 5 * j) for j, r in enumerate(batch)]     # unequal decode lengths
        heads = [len(r) - k for r, k in zip(batch, tails)]
        out = model.step(small, [StepEntry(s, r[:h], list(range(h))) for s, r, h in zip(seqs, batch, heads)])
        at = 0
        for j, (r, h) in enumerate(zip(batch, heads)):
            ref = refs[reqs.index(r)]
            assert_close(out[at:at + h], ref[:h], dtype, f"batched prefill: batch {bi} request {j}")
            at += h
        done = [0] * len(batch)
        live = [j for j in range(len(batch)) if tails[j] > 0]
        for j in range(len(batch)):
            if tails[j] == 0:
                small.close_sequence(seqs[j])
        while live:
            out = model.step(small, [StepEntry(seqs[j], [batch[j][heads[j] + done[j]]]) for j in live])
            for row, j in enumerate(live):
                ref = refs[reqs.index(batch[j])]
                assert_close(out[row], ref[heads[j] + done[j]], dtype,
                             f"batched decode: batch {bi} request {j} position {heads[j] + done[j]}")
                done[j] += 1
            for j in list(live):
                if done[j] == tails[j]:
                    small.close_sequence(seqs[j])           # ends earlier than its neighbours
                    live.remove(j)
                    small.fill_free_pages(float("nan"))     # what it held must not matter any more
        small.check()
    assert small.slots.n_held == 0 and all(g.pages.n_held == 0 for g in small.kv_groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["B", "C"])
def test_wanting_some_rows_changes_no_logit_and_no_cache(tmp, which, dtype):
    """When logits are wanted at some rows only, the last layer hands on those rows alone.  The logits
    must be those of a step that wants every row, in the order asked for (also out of order and twice),
    every token must still reach the cache (decoding on from either step gives the same logits), and
    two prompts in one step must each get their own rows."""
    from dotllm_b200 import StepEntry
    model, cfg, weights, _ = load_pair(tmp, which, dtype)
    a = tiny_models.random_tokens(150, cfg["vocab_size"], seed=31)
    b = tiny_models.random_tokens(70, cfg["vocab_size"], seed=32)
    ref_a, ref_b = plain_llama.forward(cfg, weights, list(a) + [5, 6]), plain_llama.forward(cfg, weights, b)
    cache = model.new_cache(max_tokens=1024)
    cache.fill_free_pages(float("nan"))
    s_all, s_some, s_b = cache.open_sequence(), cache.open_sequence(), cache.open_sequence()
    everything = model.step(cache, [StepEntry(s_all, a, list(range(len(a))))])
    wants = [149, 3, 64, 3, 0]
    some = model.step(cache, [StepEntry(s_some, a, wants), StepEntry(s_b, b, [69, 10])])
    assert some.shape[0] == len(wants) + 2
    assert_close(some[:len(wants)], ref_a[wants], dtype, "wanted rows of the first prompt")
    assert_close(some[len(wants):], ref_b[[69, 10]], dtype, "wanted rows of the second prompt")
    if dtype == torch.float32:      # one kernel whatever the number of rows: the same bits
        assert torch.equal(some[:len(wants)], everything[wants])
    # the cache holds every token of both steps: two more tokens give the plain logits from either
    for s in (s_all, s_some):
        out = torch.cat([model.step(cache, [StepEntry(s, [5])]), model.step(cache, [StepEntry(s, [6])])])
        assert_close(out, ref_a[150:152], dtype, "decoding on after the prompt")
    # no rows wanted at all: nothing returned, the cache still filled
    s_none = cache.open_sequence()
    assert model.step(cache, [StepEntry(s_none, a, [])]).shape[0] == 0
    assert_close(model.step(cache, [StepEntry(s_none, [5])]), ref_a[150:151], dtype, "after a prompt that wanted nothing")
    for s in (s_all, s_some, s_b, s_none):
        cache.close_sequence(s)
    cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_float32_cuts_give_the_same_bits(tmp, dtype):
    """In float32 every kernel's order of operations for a position is fixed, so whole, one by one
    and batched give identical bits.  (bfloat16 uses library products whose rounding depends on
    the number of rows, so it is only close.)"""
    if dtype != torch.float32:
        pytest.skip("bit equality holds for the float32 path only")
    from dotllm_b200 import StepEntry
    model, cfg, _, _ = load_pair(tmp, "B", dtype)
    a = tiny_models.random_tokens(90, cfg["vocab_size"], 1)
    b = tiny_models.random_tokens(50, cfg["vocab_size"], 2)
    cache = model.new_cache(512)
    s = cache.open_sequence()
    whole = model.step(cache, [StepEntry(s, a, list(range(90)))])
    cache.close_sequence(s)
    s1, s2 = cache.open_sequence(), cache.open_sequence()
    got = [model.step(cache, [StepEntry(s2, b[:20], []), StepEntry(s1, a[:60], list(range(60)))])]
    for t in range(60, 90):
        got.append(model.step(cache, [StepEntry(s2, [b[t - 40]], []), StepEntry(s1, [a[t]])]))
    assert torch.equal(torch.cat(got).cpu(), whole.cpu())


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_and_first_tokens(tmp, dtype):
    """One token at a time from position 0 to the model's last position (past the rope scaling's
    original length, across page boundaries)."""
    from dotllm_b200 import StepEntry
    model, cfg, weights, _ = load_pair(tmp, "B", dtype)
    n = cfg["max_position_embeddings"]
    toks = tiny_models.random_tokens(n, cfg["vocab_size"], 5)
    ref = plain_llama.forward(cfg, weights, toks)
    cache = model.new_cache(n)
    s = cache.open_sequence()
    for t in range(n):
        out = model.step(cache, [StepEntry(s, [toks[t]])])
        assert_close(out[0], ref[t], dtype, f"decode position {t}")
    from dotllm_b200.errors import StepError
    with pytest.raises(StepError):
        model.step(cache, [StepEntry(s, [0])])              # beyond max positions
    cache.close_sequence(s)


def test_far_key_decides_the_next_token(tmp):
    """Weights made so that a far key matters: scale one layer's query and key projections so the
    scores are sharp.  A cache or mask fault at a far position then changes logits by O(1)."""
    from dotllm_b200 import Model, StepEntry
    from dotllm_b200.weights import SafetensorsFile, save_safetensors
    folder = tiny_models.make_folder(tmp, "C", seed=3, dtype=torch.float32)
    with SafetensorsFile(folder / "model.safetensors") as f:
        tensors = {n: f.tensor(n).clone() for n in f.names()}
    for name in tensors:
        if "q_proj" in name or "k_proj" in name:
            tensors[name] *= 12.0
    sharp = tmp / "sharp_C"
    sharp.mkdir(exist_ok=True)
    save_safetensors(sharp / "model.safetensors", tensors)
    (sharp / "config.json").write_text((folder / "config.json").read_text())
    cfg, weights = plain_llama.read_model_folder(sharp)
    toks = tiny_models.random_tokens(600, cfg["vocab_size"], 9)
    ref = plain_llama.forward(cfg, weights, toks)
    for dtype in (torch.float32,):
        model = Model.load(sharp, dtype=dtype)
        cache = model.new_cache(1024)
        s = cache.open_sequence()
        out = [model.step(cache, [StepEntry(s, toks[:570], [0, 1, 63, 64, 569])])]
        out += [model.step(cache, [StepEntry(s, [toks[t]])]) for t in range(570, 600)]
        out = torch.cat(out)
        want = ref[[0, 1, 63, 64, 569] + list(range(570, 600))]
        err = float((out.cpu() - want).abs().max())
        assert err < 5e-4, err


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["A", "B"])
def test_greedy_generation_through_the_entry_point(tmp, which, dtype):
    from dotllm_b200 import InferenceOptions, Model
    model, cfg, weights, folder = load_pair(tmp, which, dtype)
    lens = tiny_models.TINY_A_PROMPTS if which == "A" else tiny_models.TINY_B_PROMPTS
    n_new = tiny_models.TINY_A_DECODE if which == "A" else tiny_models.TINY_B_DECODE
    prompts = [tiny_models.random_tokens(n, cfg["vocab_size"], 40 + n) for n in lens]
    opts = InferenceOptions(temperature=0.0, max_tokens=n_new, stop_token_ids=[])
    outs = model.generate(prompts, opts)
    for p, o in zip(prompts, outs):
        assert o.finish_reason.value == "length" and o.generated_token_count == n_new
        # teacher-forced check: every generated token is the plain argmax, or ties it within tolerance
        ref = plain_llama.forward(cfg, weights, p + o.generated_token_ids)
        for i, tok in enumerate(o.generated_token_ids):
            row = ref[len(p) - 1 + i]
            assert greedy_ok(row, tok, dtype), (i, tok, int(row.argmax()), float(row.max() - row[tok]))
    if dtype == torch.float32:
        for p, o in zip(prompts, outs):
            want, _ = plain_llama.greedy_generate(cfg, weights, p, n_new)
            assert o.generated_token_ids == want
    # a stop token ends a request early, is not returned, and frees its slot
    stop = outs[0].generated_token_ids[2]
    o = model.generate(prompts[0], InferenceOptions(temperature=0.0, max_tokens=n_new, stop_token_ids=[stop]))
    assert o.finish_reason.value == "stop"
    assert o.generated_token_ids == outs[0].generated_token_ids[:outs[0].generated_token_ids.index(stop)]
    # one request alone gives what it gave in the batch
    alone = model.generate(prompts[-1], opts)
    if dtype == torch.float32:
        assert alone.generated_token_ids == outs[-1].generated_token_ids


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which,n_seqs", [("A", 40), ("D", 64), ("C", 33)])
@pytest.mark.parametrize("graphs", [False, True, "shared"])
def test_decoding_many_sequences_at_once(tmp, which, n_seqs, dtype, graphs):
    """Decode steps of 33, 40 and 64 sequences of unequal lengths that end at different steps (the
    batch shrinks through 17 and 16 rows, where the decode products change kernels), eagerly, through
    a captured graph per batch size, and through graphs of a few widths whose other rows
    are idle ("shared": the idle page is poisoned, so an idle row that reached a live one would
    show); every logit against the plain implementation."""
    from dotllm_b200 import StepEntry
    model, cfg, weights, _ = load_pair(tmp, which, dtype)
    vocab, positions = cfg["vocab_size"], cfg["max_position_embeddings"]
    lens = [min(positions - 14, 3 + (37 * i) % 90 + (130 if i % 11 == 0 else 0)) for i in range(n_seqs)]
    n_decode = [2 + (5 * i) % 11 for i in range(n_seqs)]               # 2 to 12 decoded tokens each
    reqs = [tiny_models.random_tokens(n + d, vocab, seed=900 + i) for i, (n, d) in enumerate(zip(lens, n_decode))]
    refs = [plain_llama.forward(cfg, weights, r) for r in reqs]
    cache = model.new_cache(max_tokens=sum((len(r) + 63) // 64 * 64 for r in reqs))
    cache.fill_free_pages(float("nan"))
    seqs = [cache.open_sequence() for _ in reqs]
    out = model.step(cache, [StepEntry(s, r[:n]) for s, r, n in zip(seqs, reqs, lens)])
    for i, (ref, n) in enumerate(zip(refs, lens)):
        assert_close(out[i], ref[n - 1], dtype, f"prefill of sequence {i}")
    done = [0] * n_seqs
    live = list(range(n_seqs))
    sizes = set()
    while live:
        sizes.add(len(live))
        entries = [StepEntry(seqs[i], [reqs[i][lens[i] + done[i]]]) for i in live]
        if graphs == "shared":
            for g in cache.kv_groups:
                g.k[:, cache.idle_page] = float("nan")
                g.v[:, cache.idle_page] = float("nan")
            out = model.decode_graphs(cache).run(entries, capture_after=1).clone()
            assert out.shape[0] == len(live)
        else:
            out = model.step(cache, entries, graphs=graphs).clone()
        for row, i in enumerate(live):
            assert_close(out[row], refs[i][lens[i] + done[i]], dtype,
                         f"{len(live)} live: sequence {i} position {lens[i] + done[i]}")
            done[i] += 1
        for i in list(live):
            if done[i] == n_decode[i]:
                cache.close_sequence(seqs[i])
                live.remove(i)
        cache.fill_free_pages(float("nan"))
    assert max(sizes) == n_seqs and min(sizes) <= 16 and any(16 < n <= 32 for n in sizes)
    cache.check()
    if graphs == "shared":
        runner = model.decode_graphs(cache)
        assert runner.captured and all(rows % 16 == 0 or rows in (1, 2, 4, 8) for rows in runner.captured)
        assert len(runner.captured) <= 8 < len(sizes)


def test_generation_that_loses_its_requests_one_by_one(tmp):
    """Twenty greedy requests that end three steps apart, through the generation loop without graphs,
    with graphs, and with graphs and every decode step started before the tokens of the step before
    it are on the host (float32: the same bits whatever the batch, so the tokens must be the same).
    The loop's graphs come in few widths (1, 2, 4, 8, 16, 32, 48 ...): the batch sizes 20 .. 1 share
    five or fewer.  Then the same with a stop token that some requests meet on their way: a request
    that stops has run one row of the step started ahead in vain."""
    from dotllm_b200 import InferenceOptions
    model, cfg, _, _ = load_pair(tmp, "B", torch.float32)
    prompts = [tiny_models.random_tokens(4 + (7 * i) % 23, cfg["vocab_size"], seed=300 + i) for i in range(20)]

    def run(options, use_graphs, ahead):
        cache = model.new_cache(max_tokens=20 * 128)
        generator = model.generator(cache=cache, max_batch=20, use_graphs=use_graphs, ahead=ahead)
        outs = generator.generate(prompts, options)
        cache.check()
        assert not cache.live
        return outs, generator, cache

    options = [InferenceOptions(temperature=0.0, max_tokens=10 + 3 * i, stop_token_ids=[]) for i in range(20)]
    eager, _, _ = run(options, False, False)
    assert [len(o.generated_token_ids) for o in eager] == [10 + 3 * i for i in range(20)]
    for ahead in (False, True):
        outs, generator, cache = run(options, True, ahead)
        assert [o.generated_token_ids for o in outs] == [o.generated_token_ids for o in eager], f"ahead={ahead}"
        runner = model.decode_graphs(cache)
        assert 2 <= len(runner.captured) <= 5 and set(runner.captured) <= {1, 2, 4, 8, 16, 32}
        assert (generator.ahead_steps > 30) == ahead and generator.ahead_rows_in_vain == 0
    # a stop token that request 5 meets at its thirteenth token (and others wherever they meet it)
    stop = eager[5].generated_token_ids[12]
    stopping = [InferenceOptions(temperature=0.0, max_tokens=10 + 3 * i, stop_token_ids=[stop]) for i in range(20)]
    eager, _, _ = run(stopping, False, False)
    assert eager[5].finish_reason.value == "stop" and len(eager[5].generated_token_ids) <= 12
    outs, generator, _ = run(stopping, True, True)
    assert [o.generated_token_ids for o in outs] == [o.generated_token_ids for o in eager]
    assert [o.finish_reason for o in outs] == [o.finish_reason for o in eager]
    assert generator.ahead_rows_in_vain >= 1


@pytest.mark.parametrize("which,dtype", [("B", torch.float32), ("D", torch.float32), ("B", torch.bfloat16), ("D", torch.bfloat16)])
def test_random_walks_of_steps_rollbacks_and_graph_modes(tmp, which, dtype):
    """Seeded random walks over one cache: chunks of unequal sizes for some of the sequences, decode
    steps for others (eagerly, through a graph per batch size, through the loop's shared widths with
    idle rows), rollbacks to random lengths in between, NaN in every page that nobody holds.  Every
    logit that a step returns is compared with the plain implementation of the whole sequence."""
    import random
    from dotllm_b200 import StepEntry
    model, cfg, weights, _ = load_pair(tmp, which, dtype)
    vocab, positions = cfg["vocab_size"], cfg["max_position_embeddings"]
    rng = random.Random(5)
    checked = 0
    for trial in range(4):
        n = rng.randint(1, 6)
        cache = model.new_cache(max_tokens=n * ((positions + 63) // 64 * 64), max_sequences=n)
        cache.fill_free_pages(float("nan"))
        full = [tiny_models.random_tokens(rng.randint(20, min(positions, 230)), vocab, seed=rng.randint(0, 10 ** 6)) for _ in range(n)]
        refs = [plain_llama.forward(cfg, weights, f) for f in full]
        seqs = [cache.open_sequence() for _ in range(n)]
        for op in range(40):
            live = [i for i in range(n) if seqs[i].length < len(full[i])]
            if not live:
                break
            kind = rng.random()
            if kind < 0.15:                                              # roll a sequence back
                i = rng.randrange(n)
                if seqs[i].length > 1:
                    cache.truncate(seqs[i], rng.randint(1, seqs[i].length))
                    cache.fill_free_pages(float("nan"))
                continue
            started = [i for i in live if seqs[i].length > 0]
            if kind < 0.65 and started:                                  # one token each
                chosen = rng.sample(started, rng.randint(1, len(started)))
                entries = [StepEntry(seqs[i], [full[i][seqs[i].length]]) for i in chosen]
                wanted = [(i, seqs[i].length) for i in chosen]
                mode = rng.choice([False, True, "lazy", "shared"])
                if mode == "shared":
                    out = model.decode_graphs(cache).run(entries, capture_after=1).clone()
                else:
                    out = model.step(cache, entries, graphs=mode).clone()
            else:                                                        # chunks of unequal sizes
                chosen = rng.sample(live, rng.randint(1, len(live)))
                entries, wanted, mode = [], [], "chunks"
                for i in chosen:
                    start = seqs[i].length
                    size = min(rng.choice([1, 2, 7, 33, 64, 70]), len(full[i]) - start)
                    entries.append(StepEntry(seqs[i], full[i][start:start + size], [0, size - 1] if size > 1 else [0]))
                    wanted += [(i, start), (i, start + size - 1)] if size > 1 else [(i, start)]
                out = model.step(cache, entries, graphs=rng.choice([False, True])).clone()
            assert out.shape[0] == len(wanted)
            for row, (i, p) in enumerate(wanted):
                assert_close(out[row], refs[i][p], dtype, f"walk {trial}, step {op} ({mode}): sequence {i}, position {p}")
                checked += 1
        cache.check()
    assert checked > 100


@pytest.mark.parametrize("which", ["A", "D"])
def test_random_generation_workloads_give_the_same_tokens_whatever_the_loop_does(tmp, which):
    """Seeded random workloads (1 to 40 requests, greedy or drawn with a repetition penalty, with and
    without stop tokens that some requests meet, batches cut by a batch limit) through the loop
    without graphs, with graphs of shared widths, and with steps started ahead; every workload twice,
    so that the second call meets its graphs from the first step on.  float32: the same tokens and
    the same reasons to end; nothing is left in the cache."""
    import random
    from dotllm_b200 import InferenceOptions
    model, cfg, _, _ = load_pair(tmp, which, torch.float32)
    vocab, positions = cfg["vocab_size"], cfg["max_position_embeddings"]
    rng = random.Random(11)
    for trial in range(6):
        n = rng.choice([1, 3, 9, 17, 24, 40])
        prompts = [tiny_models.random_tokens(rng.randint(1, min(60, positions // 3)), vocab, seed=rng.randint(0, 10 ** 6))
                   for _ in range(n)]
        stops = [rng.randrange(vocab) for _ in range(rng.choice([0, 3, 12]))]
        drawn = trial % 2 == 1
        options = [InferenceOptions(temperature=0.9 if drawn else 0.0, top_k=20 if drawn else 0, seed=rng.randint(0, 999),
                                    repetition_penalty=rng.choice([1.0, 1.3]), max_tokens=rng.randint(1, min(70, positions - 61)),
                                    stop_token_ids=stops) for _ in range(n)]
        max_batch = rng.choice([n, max(1, n // 2)])
        outs = {}
        for mode, (use_graphs, ahead) in {"eager": (False, False), "graphs": (True, False), "ahead": (True, True)}.items():
            cache = model.new_cache(max_tokens=max(n, 4) * 192)
            generator = model.generator(cache=cache, max_batch=max_batch, use_graphs=use_graphs, ahead=ahead)
            for _ in range(2):
                results = generator.generate(prompts, options)
            outs[mode] = [(r.generated_token_ids, r.finish_reason) for r in results]
            cache.check()
            assert not cache.live
        assert outs["graphs"] == outs["eager"], f"trial {trial}: graphs"
        assert outs["ahead"] == outs["eager"], f"trial {trial}: steps ahead"


def test_a_sampled_request_gives_the_same_tokens_alone_and_in_any_batch(tmp):
    """A request's draws depend on its own seed and step only: the same prompt, options and seed give
    the same tokens alone, as the first of a batch and as the last of another (float32, where the
    logits do not depend on the batch either)."""
    from dotllm_b200 import InferenceOptions
    model, cfg, _, _ = load_pair(tmp, "A", torch.float32)
    vocab = cfg["vocab_size"]
    mine = tiny_models.random_tokens(12, vocab, 77)
    others = [tiny_models.random_tokens(n, vocab, 80 + n) for n in (5, 20, 9)]
    o_mine = InferenceOptions(temperature=0.8, top_k=40, top_p=0.9, seed=1234, max_tokens=12, stop_token_ids=[])
    o_other = InferenceOptions(temperature=1.1, seed=99, max_tokens=7, stop_token_ids=[])
    alone = model.generate(mine, o_mine).generated_token_ids
    first = model.generate([mine] + others, [o_mine] + [o_other] * 3)[0].generated_token_ids
    last = model.generate(others + [mine], [o_other] * 3 + [o_mine])[3].generated_token_ids
    assert alone == first == last
    # the same seed on two requests of one batch: the same stream for both (they differ by their logits only)
    twice = model.generate([mine, mine], o_mine)
    assert twice[0].generated_token_ids == twice[1].generated_token_ids == alone


def test_seeded_sampling_is_reproducible_and_batch_independent(tmp):
    from dotllm_b200 import InferenceOptions
    model, cfg, _, _ = load_pair(tmp, "A", torch.float32)
    prompts = [tiny_models.random_tokens(n, cfg["vocab_size"], 70 + n) for n in (6, 13, 9)]
    opts = [InferenceOptions(temperature=0.9, top_k=50, top_p=0.95, seed=11 + i, max_tokens=10, stop_token_ids=[])
            for i in range(3)]
    a = model.generate(prompts, opts)
    b = model.generate(prompts, opts)
    assert [o.generated_token_ids for o in a] == [o.generated_token_ids for o in b]
    different = model.generate(prompts, [InferenceOptions(temperature=0.9, seed=99, max_tokens=10, stop_token_ids=[])] * 3)
    assert [o.generated_token_ids for o in different] != [o.generated_token_ids for o in a]


@pytest.mark.parametrize("which", ["A", "B"])
def test_dependent_launch_changes_no_bit(tmp, which):
    """Kernels that may begin before the kernel ahead of them has finished give the same logits,
    bit for bit, as the same kernels launched strictly one after another - eagerly and from
    captured graphs."""
    from dotllm_b200 import StepEntry
    from dotllm_b200.kernels import library
    model, cfg, _, _ = load_pair(tmp, which, torch.bfloat16)
    prompts = [tiny_models.random_tokens(n, cfg["vocab_size"], seed=300 + n) for n in (70, 9, 100)]
    follow = [tiny_models.random_tokens(12, cfg["vocab_size"], seed=400 + i) for i in range(3)]

    def run(dependent, graphs):
        library.set_dependent_launch(dependent)
        try:
            cache = model.new_cache(max_tokens=1024)
            seqs = [cache.open_sequence() for _ in prompts]
            outs = [model.step(cache, [StepEntry(s, p, [len(p) - 1]) for s, p in zip(seqs, prompts)])]
            for t in range(12):
                outs.append(model.step(cache, [StepEntry(s, [f[t]]) for s, f in zip(seqs, follow)], graphs=graphs))
            for s in seqs:
                cache.close_sequence(s)
            return torch.cat(outs).clone()
        finally:
            library.set_dependent_launch(True)

    for graphs in (False, True):
        base = run(False, graphs)
        got = run(True, graphs)
        assert torch.equal(got, base), f"graphs={graphs}: max diff {(got - base).abs().max()}"
        again = run(True, graphs)
        assert torch.equal(got, again), f"graphs={graphs}: two runs differ by {(got - again).abs().max()}"


def test_graph_steps_staged_ahead_follow_what_the_caller_does(tmp):
    """After a captured decode step the next step's positions, lengths and tables are sent ahead for the
    same sequences.  The guess must be dropped when the caller does something else: crosses a page,
    swaps a sequence for another of the same length, truncates one, or runs an eager step in between.
    In float32 every cut gives the same bits, so graphs are compared with eager steps exactly."""
    from dotllm_b200 import StepEntry
    model, cfg, _, _ = load_pair(tmp, "A", torch.float32)
    vocab = cfg["vocab_size"]
    prompts = [tiny_models.random_tokens(n, vocab, seed=500 + n) for n in (61, 30, 61)]
    feed = [tiny_models.random_tokens(40, vocab, seed=600 + i) for i in range(3)]

    def run(graphs):
        cache = model.new_cache(max_tokens=1024)
        seqs = [cache.open_sequence() for _ in prompts]
        outs = [model.step(cache, [StepEntry(s, p, [len(p) - 1]) for s, p in zip(seqs, prompts)])]
        # a graph's logits live in a buffer that its next replay overwrites: keep copies
        two = lambda t, a, b: model.step(cache, [StepEntry(seqs[a], [feed[a][t]]), StepEntry(seqs[b], [feed[b][t]])],
                                         graphs=graphs).clone()
        for t in range(6):                                  # 0 and 1 together; sequence 0 crosses a page at its 65th token
            outs.append(two(t, 0, 1))
        for t in range(6, 9):                               # same batch size and slot order, but 2 (as long as 0 was) for 0
            outs.append(two(t, 2, 1))
        outs.append(two(9, 0, 1))                           # back again
        cache.truncate(seqs[1], seqs[1].length - 2)         # 1 goes two tokens back and on from there
        for t in range(10, 14):
            outs.append(two(t, 0, 1))
        outs.append(model.step(cache, [StepEntry(seqs[0], [feed[0][14]]), StepEntry(seqs[1], [feed[1][14]])]))   # an eager step
        for t in range(15, 18):
            outs.append(two(t, 0, 1))
        cache.check()
        if graphs:
            # of the 17 graph steps, those straight after another one of the same two sequences at the next
            # length find everything but their tokens on the device: not the first, not after a swap, the
            # truncation or the eager step, and not the two steps that need a new page
            assert model.decode_graphs(cache).ahead_hits == 11
        for s in seqs:
            cache.close_sequence(s)
        return torch.cat(outs).clone()

    eager, graphed = run(False), run(True)
    assert torch.equal(eager, graphed), f"max diff {(eager - graphed).abs().max()}"


def test_graph_step_after_pages_changed_at_the_same_length(tmp):
    """Two sequences are truncated by more than a page and grown back, by an eager step, to the very
    length for which the graph's tables were sent ahead.  The cache hands out the most recently freed
    page first, so the two sequences come back holding each other's old pages: a graph step that
    trusted the tables sent ahead would write into, and read from, the other sequence's page."""
    from dotllm_b200 import StepEntry
    model, cfg, _, _ = load_pair(tmp, "A", torch.float32)
    vocab = cfg["vocab_size"]
    prompts = [tiny_models.random_tokens(70, vocab, seed=700 + i) for i in range(2)]
    feed = [tiny_models.random_tokens(80, vocab, seed=710 + i) for i in range(2)]

    def run(graphs):
        cache = model.new_cache(max_tokens=512)
        seqs = [cache.open_sequence() for _ in prompts]
        outs = [model.step(cache, [StepEntry(s, p, [len(p) - 1]) for s, p in zip(seqs, prompts)])]
        one = lambda t, g: model.step(cache, [StepEntry(s, [f[t]]) for s, f in zip(seqs, feed)], graphs=g).clone()
        for t in range(3):
            outs.append(one(t, graphs))                     # lengths 73; the step for 73 -> 74 is sent ahead
        before = [list(s.pages[0]) for s in seqs]
        for s in seqs:
            cache.truncate(s, 3)                            # gives back the second page of each
        regrow = [p[3:] + f[:3] for p, f in zip(prompts, feed)]
        outs.append(model.step(cache, [StepEntry(s, r) for s, r in zip(seqs, regrow)]))     # eager, back to 73
        assert [s.length for s in seqs] == [73, 73]
        assert [list(s.pages[0]) for s in seqs] != before   # the point of the test: other pages, same lengths
        for t in range(3, 6):
            outs.append(one(t, graphs))
        cache.check()
        for s in seqs:
            cache.close_sequence(s)
        return torch.cat(outs).clone()

    eager, graphed = run(False), run(True)
    assert torch.equal(eager, graphed), f"max diff {(eager - graphed).abs().max()}"


REAL_SIZES = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 131072, "hidden_act": "silu",
}


def test_two_layers_at_the_benchmark_models_sizes(tmp_path):
    """Two layers with the layer sizes of the benchmark model (hidden 4096, 32 / 8 heads of 128,
    feed-forward 14336, vocabulary 128256): three unequal prompts that cross page boundaries in one
    step, then eight decode steps, in float32 (bound 1e-3 and the plain implementation's arg-max at
    every step) and in bfloat16, every logit against the plain implementation.  The kernels run at
    the sizes they are tuned for, which the tiny models never reach (cut tiles in the products, the
    tcgen05 prefill attention, the LM head's 1002 tiles)."""
    from dotllm_b200 import Model, StepEntry
    from dotllm_b200.config import config_from_dict
    from dotllm_b200.weights import write_random_model
    folder = write_random_model(tmp_path / "real", config_from_dict(REAL_SIZES), seed=21, dtype=torch.bfloat16)
    cfg, weights = plain_llama.read_model_folder(folder)       # bfloat16 numbers widened to float32: both sides read the same
    vocab, n_new = cfg["vocab_size"], 8
    prompts = [tiny_models.random_tokens(n, vocab, seed=50 + n) for n in (70, 130, 193)]

    def plain_rows(tokens, rows):
        """Plain logits of ``tokens`` at ``rows`` only (the head over 128256 outputs is the costly part)."""
        cos, sin = plain_llama.rope_tables(range(len(tokens)), cfg["head_dim"], cfg["rope_theta"], cfg["rope_scaling"])
        h = plain_llama.embed(weights["model.embed_tokens.weight"], tokens)
        for layer in range(cfg["num_hidden_layers"]):
            h = plain_llama.block(h, weights, layer, cfg, cos, sin)
        h = plain_llama.rms_norm(h[rows], weights["model.norm.weight"], cfg["rms_norm_eps"])
        return plain_llama.linear(h, weights["lm_head.weight"])

    forced = None
    # bfloat16 at these sizes: the plain implementation itself, with its activations rounded to bfloat16
    # between parts, moves by 7.1e-2 at most and by 1.1e-2 of a row's rms (the embedding's rows are
    # tiny, so the stream is made of branch outputs and their rounding); the engine shows 7.5e-2 and 1.3e-2.
    for dtype, bound, rel_bound in ((torch.float32, 1e-3, 1e-4), (torch.bfloat16, 0.15, 2.5e-2)):
        model = Model.load(folder, dtype=dtype)
        cache = model.new_cache(max_tokens=1024)
        seqs = [cache.open_sequence() for _ in prompts]
        got = [model.step(cache, [StepEntry(s, p) for s, p in zip(seqs, prompts)]).cpu()]
        if forced is None:
            # float32 first: its own greedy tokens are the continuation, checked against the plain arg-max below
            tokens = [[int(t)] for t in got[0].argmax(dim=-1)]
            for step in range(1, n_new):
                got.append(model.step(cache, [StepEntry(s, [t[-1]]) for s, t in zip(seqs, tokens)]).cpu())
                for t, row in zip(tokens, got[-1]):
                    t.append(int(row.argmax()))
            forced = tokens
        else:
            # bfloat16: the forced continuation, first through the loop's graph of four rows with an idle
            # one (an eager step, the capture, two replays), then through the graph of three rows
            for step in range(1, n_new):
                entries = [StepEntry(s, [t[step - 1]]) for s, t in zip(seqs, forced)]
                if step <= 4:
                    got.append(model.decode_graphs(cache).run(entries, capture_after=1).cpu().clone())
                else:
                    got.append(model.step(cache, entries, graphs=True).cpu().clone())
            assert set(model.decode_graphs(cache).captured) == {3, 4}
        for s in seqs:
            cache.close_sequence(s)
        del model, cache
        torch.cuda.empty_cache()
        worst = 0.0
        for i, (p, cont) in enumerate(zip(prompts, forced)):
            rows = [len(p) - 1 + j for j in range(n_new)]
            ref = plain_rows(p + cont[:n_new - 1], rows)
            mine = torch.stack([g[i] for g in got])
            err = float((mine - ref).abs().max())
            worst = max(worst, err)
            rel = float(((mine - ref).norm(dim=1) / ref.norm(dim=1)).max())
            assert rel <= rel_bound, f"{dtype}: request {i}: a row's rms error is {rel:.3e} of its rms"
            assert err <= bound, f"{dtype}: request {i} differs from the plain implementation by {err:.3e}"
            if dtype == torch.float32:
                assert [int(r.argmax()) for r in ref] == cont, f"request {i}: greedy tokens differ from the plain arg-max"
        print(f"real sizes {dtype}: max |logit difference| {worst:.3e}")


@pytest.mark.parametrize("which", ["B", "D"])
def test_a_captured_prompt_step_keeps_what_it_copies_from_the_host(tmp, which):
    """The bfloat16 prefill attention gets its list of tiles from the host inside the step; a captured
    step copies it again at every replay, from the same pinned memory.  That memory must stay the
    step's own: here another step with as many tiles in another order runs between the capture and
    the replay, and small pinned buffers come and go.  The replay must give the eager step's bits."""
    from dotllm_b200 import StepEntry
    model, cfg, _, _ = load_pair(tmp, which, torch.bfloat16)
    vocab = cfg["vocab_size"]
    lens, other = (200, 9, 33), (9, 33, 200)

    def step(cache, sizes, seed, graphs):
        seqs = [cache.open_sequence() for _ in sizes]
        prompts = [tiny_models.random_tokens(n, vocab, seed=seed + i) for i, n in enumerate(sizes)]
        out = model.step(cache, [StepEntry(s, p, [0, len(p) - 1]) for s, p in zip(seqs, prompts)], graphs=graphs).clone()
        for s in seqs:
            cache.close_sequence(s)
        return out

    cache = model.new_cache(max_tokens=2048)
    want = step(cache, lens, 30, False)
    cache = model.new_cache(max_tokens=2048)
    step(cache, lens, 10, True)                                  # seen once: eager
    step(cache, lens, 20, True)                                  # seen twice: captured
    assert model.step_graphs(cache).captures == 1
    step(cache, other, 40, False)                                # as many tiles, in another order
    churn = [torch.full((n,), 7, dtype=torch.int32).pin_memory() for n in (4, 8, 12, 16, 24, 32, 64) for _ in range(4)]
    del churn
    got = step(cache, lens, 30, True)                            # replayed
    assert model.step_graphs(cache).replays == 1
    assert torch.equal(got, want), f"max diff {(got - want).abs().max()}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompts_of_other_lengths_share_a_captured_step(tmp, dtype):
    """A captured prompt step runs at a length that several prompt lengths share (the next multiple
    of 64, a power of two below): the tokens that fill it up come after the prompt's own, so no
    wanted row sees them, and the cache forgets them after the step.  Prompts of 70, 100, 90, 128 and
    65 tokens, and batches of three, through one graph each; then decode steps from what the cache
    holds.  float32: the bits of eager steps.  bfloat16: against the plain implementation."""
    from dotllm_b200 import StepEntry
    model, cfg, weights, _ = load_pair(tmp, "D", dtype)
    vocab = cfg["vocab_size"]
    singles = [[n] for n in (70, 100, 90, 128, 65)]
    batches = [[70, 9, 33], [100, 12, 40], [65, 16, 64], [128, 10, 50]]

    def run(graphs):
        cache = model.new_cache(max_tokens=64 * 16)
        outs, seed = [], 0
        for sizes in singles + batches:
            seqs = [cache.open_sequence() for _ in sizes]
            reqs = [tiny_models.random_tokens(n + 3, vocab, seed=7000 + (seed := seed + 1)) for n in sizes]
            entries = [StepEntry(s, r[:n], [0, n - 1]) for s, r, n in zip(seqs, reqs, sizes)]
            outs.append((reqs, [p for n in sizes for p in (0, n - 1)], model.step(cache, entries, graphs=graphs).clone()))
            assert [s.length for s in seqs] == list(sizes)
            assert [len(s.pages[cache.kv_groups[0].index]) for s in seqs] == [(n + 63) // 64 for n in sizes]
            for t in range(3):                                   # the cache holds the prompt and nothing else
                step = model.step(cache, [StepEntry(s, [r[n + t]]) for s, r, n in zip(seqs, reqs, sizes)]).clone()
                outs.append((reqs, [n + t for n in sizes], step))
            for s in seqs:
                cache.close_sequence(s)
            cache.check()
        if graphs:
            g = model.step_graphs(cache)
            assert g.captures == 2 and g.replays == 3 + 2        # one graph for the singles, one for the batches
        return outs

    graphed = run(True)
    if dtype == torch.float32:
        eager = run(False)
        for (_, _, a), (_, _, b) in zip(eager, graphed):
            assert torch.equal(a, b), f"max diff {(a - b).abs().max()}"
    for reqs, positions, got in graphed:
        refs = [plain_llama.forward(cfg, weights, r) for r in reqs]
        per = len(positions) // len(reqs)
        for row, p in enumerate(positions):
            assert_close(got[row], refs[row // per][p], dtype, f"position {p} of a request of {len(reqs[row // per])} tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_chunks_that_continue_a_sequence_share_captured_steps(tmp, dtype):
    """One to three sequences brought in four chunks each (64 tokens, then 33 - 64, 5 - 8 and 65 - 128
    more): the chunk lengths of a round share captured steps with the rounds before and with each
    other (64, 64, 8, 128 rows a sequence; where a chunk starts is data of the step), a chunk's filling
    lies beyond its own tokens and is forgotten before the next chunk starts where the sequence
    really ends.  Three logits of every chunk against the plain
    implementation of the whole sequence."""
    import random
    from dotllm_b200 import StepEntry
    model, cfg, weights, _ = load_pair(tmp, "D", dtype)
    vocab = cfg["vocab_size"]
    rng = random.Random(9)
    cache = model.new_cache(max_tokens=64 * 24)
    for trial in range(8):
        n = 1 + trial % 3
        sizes = [[64, rng.randint(33, 64), rng.randint(5, 8), rng.randint(65, 128)] for _ in range(n)]
        full = [tiny_models.random_tokens(sum(s), vocab, seed=rng.randint(0, 10 ** 6)) for s in sizes]
        refs = [plain_llama.forward(cfg, weights, f) for f in full]
        seqs = [cache.open_sequence() for _ in range(n)]
        for c in range(4):
            entries, wanted = [], []
            for i in range(n):
                start, size = seqs[i].length, sizes[i][c]
                entries.append(StepEntry(seqs[i], full[i][start:start + size], [0, size // 2, size - 1]))
                wanted += [(i, start), (i, start + size // 2), (i, start + size - 1)]
            out = model.step(cache, entries, graphs=True).clone()
            for row, (i, p) in enumerate(wanted):
                assert_close(out[row], refs[i][p], dtype, f"round {trial}, chunk {c}: sequence {i}, position {p}")
            assert [s.length for s in seqs] == [sum(sizes[i][:c + 1]) for i in range(n)]
        for s in seqs:
            cache.close_sequence(s)
        cache.check()
    g = model.step_graphs(cache)
    # three batch sizes, three chunk lengths each (64, 8 and 128 rows a sequence: where a chunk starts is data)
    assert g.captures == 9 and g.replays == 14


def test_prompt_steps_replayed_from_graphs_of_their_shape(tmp):
    """A step of any shape is captured when its shape comes a second time and replayed from then on:
    the same bits as eager steps (float32), for other tokens, other slots and other pages than the
    captured ones, with the least recently used graph dropped beyond the capacity."""
    from dotllm_b200 import StepEntry
    model, cfg, _, _ = load_pair(tmp, "B", torch.float32)
    vocab = cfg["vocab_size"]

    def run(graphs):
        cache = model.new_cache(max_tokens=2048)
        outs = []
        for rnd in range(4):                                 # the same two shapes four times, with other tokens
            seqs = [cache.open_sequence() for _ in range(3)]
            if rnd % 2:
                seqs = seqs[::-1]                            # other slots and pages under the same shape
            prompts = [tiny_models.random_tokens(n, vocab, seed=1000 + 10 * rnd + i) for i, n in enumerate((70, 9, 33))]
            outs.append(model.step(cache, [StepEntry(s, p, [0, len(p) - 1]) for s, p in zip(seqs, prompts)], graphs=graphs).clone())
            chunk = [tiny_models.random_tokens(16, vocab, seed=2000 + 10 * rnd + i) for i in range(3)]
            outs.append(model.step(cache, [StepEntry(s, c) for s, c in zip(seqs, chunk)], graphs=graphs).clone())
            outs.append(model.step(cache, [StepEntry(s, [c[0]]) for s, c in zip(seqs, chunk)], graphs=graphs).clone())
            for s in seqs:
                cache.close_sequence(s)
        cache.check()
        if graphs:
            g = model.step_graphs(cache)
            assert g.captures == 2 and g.replays == 4        # each shape: eager, captured, replayed twice
        return torch.cat(outs)

    eager, graphed = run(False), run(True)
    assert torch.equal(eager, graphed), f"max diff {(eager - graphed).abs().max()}"
