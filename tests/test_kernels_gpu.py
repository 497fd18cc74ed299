"""Each CUDA kernel alone against its plain torch reference, at sizes other than the engine's."""
import math

import pytest
import torch

import kernel_refs
import plain_llama

pytestmark = pytest.mark.gpu
DEV = "cuda"


def ops():
    from dotllm_b200.kernels import ops as o
    return o


def close(a, b, atol, rtol=0.0):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs()
    bound = atol + rtol * b.abs()
    assert bool((err <= bound).all()), f"max err {float(err.max()):.3e} (bound {atol:.1e}+{rtol:.1e}*|ref|)"


def bf16_round(x):
    return x.to(torch.bfloat16).to(torch.float32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width,vocab", [(1, 48, 7), (37, 1000, 301)])
def test_gather_rows(dtype, rows, width, vocab):
    g = torch.Generator().manual_seed(1)
    table = torch.randn(vocab, width, generator=g).to(dtype).to(DEV)
    ids = torch.randint(0, vocab, (rows,), generator=g, dtype=torch.int32).to(DEV)
    out = ops().gather_rows(table, ids)
    assert out.dtype == torch.float32
    assert torch.equal(out.cpu(), kernel_refs.gather_rows(table.cpu(), ids.cpu()))
    # rows kept in their own dtype, and rows of a table that is a column slice of a wider matrix
    same = ops().gather_rows(table, ids, out_dtype=dtype)
    assert same.dtype == dtype and torch.equal(same.cpu(), table.cpu()[ids.cpu().long()])
    wide = torch.randn(vocab, width + 24, generator=g).to(dtype).to(DEV)
    part = wide[:, 8:8 + width]
    assert torch.equal(ops().gather_rows(part, ids, out_dtype=dtype).cpu(), part.cpu()[ids.cpu().long()])
    if dtype == torch.float32:
        from dotllm_b200.errors import KernelError
        with pytest.raises(KernelError):
            ops().gather_rows(table, ids, out_dtype=torch.bfloat16)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("delta_dtype", [None, torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width,eps", [(3, 72, 1e-5), (17, 1000, 1e-6), (2, 4096, 1e-5)])
def test_add_rmsnorm(out_dtype, delta_dtype, rows, width, eps):
    g = torch.Generator().manual_seed(2)
    res = torch.randn(rows, width, generator=g) * 3
    res[0, :5] = 100.0                                   # a row with large entries
    gain = 1 + 0.1 * torch.randn(width, generator=g)
    delta = None if delta_dtype is None else torch.randn(rows, width, generator=g).to(delta_dtype)
    ref_res = res.clone()
    ref = kernel_refs.add_rmsnorm(ref_res, delta, gain, eps, torch.float32)
    d_res = res.to(DEV)
    out = ops().add_rmsnorm(d_res, None if delta is None else delta.to(DEV), gain.to(DEV), eps, out_dtype)
    assert out.dtype == out_dtype
    close(d_res, ref_res, 0, 0) if delta is None else close(d_res, ref_res, 1e-6, 1e-6)
    if out_dtype == torch.float32:
        close(out, ref, 1e-5, 1e-5)
    else:
        close(out, ref, 1e-6, 2 ** -8)


def test_rmsnorm_known_values():
    """Hand-calculated case in the manner of the reference's RmsNormTests.KnownValues_HandCalculated
    (tests/DotLLM.Tests.Unit/Cpu/Kernels/RmsNormTests.cs): x=[1,2,3,4], w=1, eps=0:
    rms = sqrt(30/4)."""
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0]], device=DEV)
    out = ops().add_rmsnorm(x, None, torch.ones(4, device=DEV), 1e-12, torch.float32)
    rms = math.sqrt(30.0 / 4.0)
    close(out, torch.tensor([[1 / rms, 2 / rms, 3 / rms, 4 / rms]]), 1e-6)
    zeros = torch.zeros(1, 8, device=DEV)               # eps keeps 0/0 away
    out = ops().add_rmsnorm(zeros, None, torch.ones(8, device=DEV), 1e-5, torch.float32)
    assert bool(torch.isfinite(out).all()) and float(out.abs().max()) == 0.0


def make_paged(n_seqs, lengths, nkv, hd, dtype, seed, n_pages=None, shuffle=True):
    """Random K/V for sequences of the given lengths scattered over pages; returns pools, the
    block table and the dense per-sequence K, V [len, nkv, hd] (already rounded to dtype)."""
    g = torch.Generator().manual_seed(seed)
    need = [(n + 63) // 64 for n in lengths]
    total = sum(need)
    n_pages = n_pages or total + 3
    order = torch.randperm(n_pages, generator=g).tolist() if shuffle else list(range(n_pages))
    width = max(need)
    table = torch.full((n_seqs, width), -1, dtype=torch.int32)
    k_pool = torch.full((n_pages, nkv, 64, hd), float("nan"))
    v_pool = torch.full((n_pages, nkv, hd, 64), float("nan"))
    dense = []
    at = 0
    for b, n in enumerate(lengths):
        k = torch.randn(n, nkv, hd, generator=g).to(dtype).float()
        v = torch.randn(n, nkv, hd, generator=g).to(dtype).float()
        dense.append((k, v))
        for p in range(need[b]):
            page = order[at]
            at += 1
            table[b, p] = page
            m = min(64, n - 64 * p)
            k_pool[page, :, :m, :] = k[64 * p:64 * p + m].permute(1, 0, 2)
            v_pool[page, :, :, :m] = v[64 * p:64 * p + m].permute(1, 2, 0)
    return k_pool.to(dtype), v_pool.to(dtype), table, dense


def dense_attention(q, k, v, nh, nkv, scale, pos, window):
    first = max(0, pos - window + 1) if window else 0
    kk = k[first:pos + 1].reshape(pos + 1 - first, -1)
    vv = v[first:pos + 1].reshape(pos + 1 - first, -1)
    return plain_llama.causal_attention(q[None].float(), kk, vv, nh, nkv, scale, position_offset=pos - first)[0]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, 0), (6, 6, 32, 0), (8, 2, 64, 0), (5, 1, 48, 0),
                                              (8, 2, 128, 0), (4, 4, 80, 0), (4, 2, 32, 37), (3, 3, 256, 100)])
def test_attention_generic(dtype, nh, nkv, hd, window):
    """Prefill chunks and decode tokens mixed in one call, unequal lengths, scattered pages with
    NaN in every unused place."""
    lengths = [1, 70, 133, 64, 200]
    news = [1, 70, 5, 1, 130]                           # tokens this "step" brings (the tail of each)
    k_pool, v_pool, table, dense = make_paged(5, lengths, nkv, hd, dtype, seed=3)
    g = torch.Generator().manual_seed(4)
    token_seq, token_pos = [], []
    for b, (n, new) in enumerate(zip(lengths, news)):
        for p in range(n - new, n):
            token_seq.append(b)
            token_pos.append(p)
    T = len(token_seq)
    q = torch.randn(T, nh * hd, generator=g).to(dtype)
    scale = 1.0 / math.sqrt(hd)
    out = ops().attention(q.to(DEV), k_pool.to(DEV), v_pool.to(DEV),
                          torch.tensor(token_seq, dtype=torch.int32, device=DEV),
                          torch.tensor(token_pos, dtype=torch.int32, device=DEV), table.to(DEV),
                          nh, nkv, hd, scale, window)
    ref = torch.stack([dense_attention(q[t], *dense[token_seq[t]], nh, nkv, scale, token_pos[t], window)
                       for t in range(T)])
    assert bool(torch.isfinite(out).all())
    if dtype == torch.float32:
        close(out, ref, 2e-6, 1e-5)
    else:
        close(out, ref, 1e-3, 2 ** -7)


def test_attention_far_key_stands_out():
    """One far key among hundreds is made to dominate the scores: the output must be its value."""
    nh, nkv, hd, n = 4, 2, 32, 700
    k_pool, v_pool, table, dense = make_paged(1, [n], nkv, hd, torch.float32, seed=5)
    k, v = dense[0]
    q = torch.randn(1, nh * hd, generator=torch.Generator().manual_seed(6))
    far = 3
    for h in range(nh):
        q[0, h * hd:(h + 1) * hd] = k[far, h // 2] * 50.0      # score ~ 50*|k|^2*scale: dominates
    out = ops().attention(q.to(DEV), k_pool.to(DEV), v_pool.to(DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                          torch.tensor([n - 1], dtype=torch.int32, device=DEV), table.to(DEV), nh, nkv, hd,
                          1 / math.sqrt(hd), 0)
    want = torch.cat([v[far, h // 2] for h in range(nh)])
    close(out[0], want, 1e-4)
    # the same query under a window that excludes the far key must not see it
    out_w = ops().attention(q.to(DEV), k_pool.to(DEV), v_pool.to(DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                            torch.tensor([n - 1], dtype=torch.int32, device=DEV), table.to(DEV), nh, nkv, hd,
                            1 / math.sqrt(hd), 64)
    ref_w = dense_attention(q[0], k, v, nh, nkv, 1 / math.sqrt(hd), n - 1, 64)
    close(out_w[0], ref_w, 1e-5, 1e-5)
    assert float((out_w[0].cpu() - want).abs().max()) > 0.1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,rd", [(4, 2, 16, 16), (6, 6, 32, 32), (8, 2, 64, 32), (3, 1, 48, 0), (8, 2, 128, 128)])
@pytest.mark.parametrize("news", [[70, 1, 3], [20, 1, 3]])
def test_rope_cache_write(dtype, nh, nkv, hd, rd, news):
    """74 tokens take the kernel that works on tiles of 64 packed tokens (the second tile mixes
    three sequences); 24 tokens take the kernel with one block per (token, head)."""
    g = torch.Generator().manual_seed(7)
    lengths = [70, 5, 130]
    token_seq, token_pos = [], []
    for b, (n, new) in enumerate(zip(lengths, news)):
        for p in range(n - new, n):
            token_seq.append(b)
            token_pos.append(p)
    T = len(token_seq)
    n_pages = 9
    table = torch.tensor([[4, 1, -1], [7, -1, -1], [0, 8, 2]], dtype=torch.int32)
    q = torch.randn(T, nh * hd, generator=g).to(dtype)
    kv = torch.randn(T, 2 * nkv * hd, generator=g).to(dtype)
    k, v = kv[:, :nkv * hd], kv[:, nkv * hd:]           # views with a wider row stride
    cos, sin = plain_llama.rope_tables(range(256), rd, 10000.0) if rd else (None, None)
    pools = [torch.zeros(n_pages, nkv, 64, hd, dtype=dtype), torch.zeros(n_pages, nkv, hd, 64, dtype=dtype)]
    ref_q = q.clone()
    ref_pools = [p.clone() for p in pools]
    seq_t, pos_t = torch.tensor(token_seq, dtype=torch.int32), torch.tensor(token_pos, dtype=torch.int32)
    kernel_refs.rope_cache_write(ref_q, k, v, cos, sin, rd, seq_t, pos_t, table, *ref_pools, nh, nkv, hd)
    d_q, d_kv = q.to(DEV), kv.to(DEV)
    d_pools = [p.to(DEV) for p in pools]
    ops().rope_cache_write(d_q, d_kv[:, :nkv * hd], d_kv[:, nkv * hd:],
                           None if cos is None else cos.to(DEV), None if sin is None else sin.to(DEV), rd,
                           seq_t.to(DEV), pos_t.to(DEV), table.to(DEV), *d_pools, nh, nkv, hd)
    tol = 1e-6 if dtype == torch.float32 else 2 ** -7
    close(d_q, ref_q, tol, tol)
    close(d_pools[0], ref_pools[0], tol, tol)
    assert torch.equal(d_pools[1].cpu(), ref_pools[1])  # V is copied, not computed


@pytest.mark.parametrize("nh,nkv,hd,K", [(4, 2, 128, 192), (8, 4, 64, 320), (2, 2, 128, 4096)])
def test_qkv_product_that_rotates_and_writes_the_cache(nh, nkv, hd, K, monkeypatch):
    """A prompt step's Q/K/V product with the rotation and the cache write in its epilogue: the rotated
    queries and every page of the cache must have the bits that the library product followed by the rope
    and cache-write kernel gives - two sequences of unequal lengths that start at different positions
    (one inside a page), rows that are no multiple of the tile, pages in another order than the tokens."""
    from dotllm_b200.kernels import gemm_tc
    monkeypatch.setattr(gemm_tc, "QKV_FUSED", True)            # off by default: the library's product is faster at the shapes met
    g = torch.Generator().manual_seed(61)
    starts, news = [70, 0], [200, 131]                         # positions 70 .. 269 and 0 .. 130
    token_seq = [0] * news[0] + [1] * news[1]
    token_pos = list(range(starts[0], starts[0] + news[0])) + list(range(starts[1], starts[1] + news[1]))
    T = len(token_seq)
    n_pages = 12
    table = torch.tensor([[9, 3, 11, 0, 5], [7, 2, 10, -1, -1]], dtype=torch.int32)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn((nh + 2 * nkv) * hd, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    cos, sin = plain_llama.rope_tables(range(512), hd, 10000.0)
    cos, sin = cos.to(DEV), sin.to(DEV)
    seq_t, pos_t = torch.tensor(token_seq, dtype=torch.int32, device=DEV), torch.tensor(token_pos, dtype=torch.int32, device=DEV)
    def pools():
        gp = torch.Generator().manual_seed(62)                  # what the pages held before must survive where nothing is written
        return [torch.randn(n_pages, nkv, 64, hd, generator=gp).to(torch.bfloat16).to(DEV),
                torch.randn(n_pages, nkv, hd, 64, generator=gp).to(torch.bfloat16).to(DEV)]
    qd, kvd = nh * hd, nkv * hd
    ref_pools = pools()
    qkv = ops().linear(x, w)
    ref_q = qkv[:, :qd].contiguous()
    ops().rope_cache_write(ref_q, qkv[:, qd:qd + kvd], qkv[:, qd + kvd:], cos, sin, hd, seq_t, pos_t, table.to(DEV), *ref_pools,
                           nh, nkv, hd)
    got_pools = pools()
    q = ops().qkv_rope_cache(x, w, cos, sin, hd, seq_t, pos_t, table.to(DEV), *got_pools, nh, nkv, hd)
    assert q is not None
    from dotllm_b200.kernels import library
    library.check_status()
    assert torch.equal(q, ref_q)
    assert torch.equal(got_pools[0], ref_pools[0]) and torch.equal(got_pools[1], ref_pools[1])
    # a decode step's few rows, a partial rotation and float32 are not its cases
    assert ops().qkv_rope_cache(x[:64], w, cos, sin, hd, seq_t[:64], pos_t[:64], table.to(DEV), *got_pools, nh, nkv, hd) is None
    assert ops().qkv_rope_cache(x, w, cos, sin, hd // 2, seq_t, pos_t, table.to(DEV), *got_pools, nh, nkv, hd) is None


def test_rope_known_rotation():
    """Position 0 changes nothing; at position 1 the pair (1, 0) of frequency 1 becomes
    (cos 1, sin 1) (cf. RoPETests.PositionZero_NoChange / KnownRotation_HandCalculated,
    tests/DotLLM.Tests.Unit/Cpu/Kernels/RoPETests.cs)."""
    hd = 4
    cos, sin = plain_llama.rope_tables(range(4), hd, 10000.0)
    q = torch.tensor([[1.0, 2.0, 0.0, 0.0], [1.0, 0.0, 0.0, 0.0]], device=DEV)
    ops().rope_cache_write(q, None, None, cos.to(DEV), sin.to(DEV), hd, None,
                           torch.tensor([0, 1], dtype=torch.int32, device=DEV), None, None, None, 1, 1, hd,
                           write_cache=False)
    close(q[0], torch.tensor([1.0, 2.0, 0.0, 0.0]), 0)
    close(q[1], torch.tensor([math.cos(1.0), 0.0, math.sin(1.0), 0.0]), 1e-7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width", [(1, 176), (33, 1000)])
def test_swiglu(dtype, rows, width):
    x = (torch.randn(rows, 2 * width, generator=torch.Generator().manual_seed(8)) * 4).to(dtype)
    out = ops().swiglu(x.to(DEV))
    ref = kernel_refs.swiglu(x.float())
    close(out, ref, 1e-6, 1e-5 if dtype == torch.float32 else 2 ** -8)


@pytest.mark.parametrize("M,N,K", [(1, 5, 3), (7, 130, 70), (64, 64, 16), (65, 257, 1001), (300, 48, 176)])
def test_gemm_f32(M, N, K):
    g = torch.Generator().manual_seed(9)
    x, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)
    y = ops().linear(x.to(DEV), w.to(DEV))
    ref = (x.double() @ w.double().T).float()
    close(y, ref, 1e-5 * math.sqrt(K), 1e-5)
    # a row's result is the same bits whatever else is in the launch
    y1 = ops().linear(x[:1].to(DEV), w.to(DEV))
    assert torch.equal(y1.cpu(), y[:1].cpu())


@pytest.mark.parametrize("M,N,K", [(1, 64, 128), (5, 200, 320), (70, 1000, 176), (2048, 384, 192)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_linear_bf16(M, N, K, out_dtype):
    g = torch.Generator().manual_seed(10)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    y = ops().linear(x.to(DEV), w.to(DEV), out_dtype=out_dtype)
    assert y.dtype == out_dtype
    ref = x.double() @ w.double().T
    close(y, ref.float(), 1e-3, 2 ** -8 if out_dtype == torch.bfloat16 else 1e-4)


def test_argmax_ties_and_sizes():
    g = torch.Generator().manual_seed(11)
    for rows, vocab in [(1, 5), (3, 1000), (9, 128256)]:
        x = torch.randn(rows, vocab, generator=g)
        x[0, vocab // 2] = 50.0
        x[0, vocab - 1] = 50.0                          # a tie: the first index wins
        out = ops().sample(x.to(DEV))
        assert out.tolist()[0] == vocab // 2
        assert out.tolist()[1:] == torch.argmax(x, dim=-1).tolist()[1:]
    # the greedy kernel cuts a row into slices for a cluster of blocks: a tie across slices, a row with
    # nothing finite, NaN beside the maximum, and a vocabulary that the slices do not divide
    x = torch.randn(4, 1003, generator=g)
    x[1, 7] = x[1, 900] = 9.0
    x[2] = float("-inf")
    x[3, 5] = float("nan")
    x[3, 600] = 8.0
    assert ops().sample(x.to(DEV)).tolist() == [int(torch.argmax(x[0])), 7, 0, 600]
    # ... and the same through the sampling kernel's own greedy branch (a temperature of 0 per row)
    zeros = torch.zeros(4, device=DEV)
    assert ops().sample(x.to(DEV), temperature=zeros, uniform=zeros).tolist() == [int(torch.argmax(x[0])), 7, 0, 600]


def _sampled_ok(row, tok, r, **kw):
    """The kernel's token is the plain sampler's, or r lies within rounding of the boundary
    between them on the plain sampler's running sum."""
    ref = plain_llama.sample(row, [], r=r, **kw)
    if tok == ref:
        return True
    x = plain_llama.apply_min_p(plain_llama.apply_top_p(plain_llama.apply_top_k(
        plain_llama.apply_temperature(row, kw.get("temperature", 1.0)), kw.get("top_k", 0)),
        kw.get("top_p", 1.0)), kw.get("min_p", 0.0))
    if not math.isfinite(float(x[tok])):
        return False
    lo, hi = plain_llama.cdf_interval(x, tok)
    return lo - 1e-5 <= r <= hi + 1e-5


@pytest.mark.parametrize("vocab", [50, 1000, 32003])
def test_sample_chain(vocab):
    g = torch.Generator().manual_seed(12)
    settings = [dict(temperature=1.0), dict(temperature=0.7), dict(temperature=1.3, top_k=5),
                dict(temperature=0.9, top_p=0.8), dict(temperature=1.0, min_p=0.1),
                dict(temperature=0.8, top_k=40, top_p=0.9, min_p=0.05), dict(temperature=2.0, top_k=1),
                dict(temperature=1.0, top_p=0.01)]
    rows = len(settings) * 4
    x = torch.randn(rows, vocab, generator=g) * 3
    u = torch.rand(rows, generator=g)
    temp = torch.tensor([settings[i % len(settings)].get("temperature", 1.0) for i in range(rows)])
    top_k = torch.tensor([settings[i % len(settings)].get("top_k", 0) for i in range(rows)], dtype=torch.int32)
    top_p = torch.tensor([settings[i % len(settings)].get("top_p", 1.0) for i in range(rows)])
    min_p = torch.tensor([settings[i % len(settings)].get("min_p", 0.0) for i in range(rows)])
    out = ops().sample(x.to(DEV), temp.to(DEV), top_k.to(DEV), top_p.to(DEV), min_p.to(DEV), u.to(DEV)).tolist()
    again = ops().sample(x.to(DEV), temp.to(DEV), top_k.to(DEV), top_p.to(DEV), min_p.to(DEV), u.to(DEV)).tolist()
    assert out == again                                 # a seeded draw is reproducible
    for i in range(rows):
        assert _sampled_ok(x[i], out[i], float(u[i]), **settings[i % len(settings)]), (i, settings[i % len(settings)])


@pytest.mark.parametrize("vocab", [8195, 32003, 128256])
def test_sample_by_a_cluster_of_blocks_gives_the_same_tokens(vocab):
    """Long rows are sampled by a cluster of blocks that keep the row in their shared memories.  Its sums
    are the same integers as the one-block kernel's, so every token must be the same: over every
    setting of the chain, greedy rows, rows with ties at the top-k threshold that straddle slices,
    NaN and -inf entries, a row with nothing finite, and draws at both ends of [0, 1)."""
    g = torch.Generator().manual_seed(vocab)
    settings = [dict(temperature=1.0), dict(temperature=0.7), dict(temperature=1.3, top_k=5),
                dict(temperature=0.9, top_p=0.8), dict(temperature=1.0, min_p=0.1),
                dict(temperature=0.8, top_k=40, top_p=0.9, min_p=0.05), dict(temperature=2.0, top_k=1),
                dict(temperature=1.0, top_p=0.01), dict(temperature=0.0), dict(temperature=1.0, top_k=600, top_p=0.97),
                dict(temperature=0.6, top_p=0.5, min_p=0.3)]
    rows = len(settings) * 6
    x = torch.randn(rows, vocab, generator=g) * 3
    x[3] = torch.round(x[3])                                   # many exact ties everywhere in the row
    x[5, :] = -4.0
    x[5, [7, vocab // 8 + 1, vocab // 2, vocab - 3]] = 2.0     # k = 40 .. cuts a run of equal values lying in several slices
    x[16, ::3] = float("nan")
    x[17, 100:] = float("-inf")
    x[20] = float("-inf")                                       # nothing finite: index 0
    x[27, vocab - 1] = 40.0                                     # all the mass in the last slice's last entry
    u = torch.rand(rows, generator=g)
    u[0], u[1], u[2] = 0.0, 0.99999994, 0.5
    pick = lambda name, default: [settings[i % len(settings)].get(name, default) for i in range(rows)]
    temp, top_p, min_p = torch.tensor(pick("temperature", 1.0)), torch.tensor(pick("top_p", 1.0)), torch.tensor(pick("min_p", 0.0))
    top_k = torch.tensor(pick("top_k", 0), dtype=torch.int32)
    args = [t.to(DEV) for t in (x, temp, top_k, top_p, min_p, u)]
    one = ops().sample(*args, split=False).tolist()
    many = ops().sample(*args, split=True).tolist()
    assert many == one, [(i, settings[i % len(settings)], a, b) for i, (a, b) in enumerate(zip(one, many)) if a != b][:5]
    assert ops().sample(*args).tolist() == one                  # whichever the library chooses
    assert one[20] == 0 and one[27] == vocab - 1
    for i in range(rows if vocab < 100000 else 0):              # and both are the plain sampler's tokens (slow on the host)
        if all(torch.isfinite(x[i])) and settings[i % len(settings)].get("temperature", 1.0) > 0:
            assert _sampled_ok(x[i], one[i], float(u[i]), **settings[i % len(settings)]), (i, settings[i % len(settings)])


def test_sample_top_k_ties_in_index_order():
    """Five logits tie at the k-th value; only the first of them (by index) may be drawn
    (src/DotLLM.Engine/Samplers/TopKSampler.cs:58-78)."""
    vocab = 300
    x = torch.full((64, vocab), -5.0)
    x[:, 10] = 3.0
    x[:, [20, 40, 60, 80, 100]] = 1.0                    # k = 3: 10, 20, 40 are kept
    u = torch.linspace(0, 0.999, 64)
    out = ops().sample(x.to(DEV), torch.ones(64, device=DEV), torch.full((64,), 3, dtype=torch.int32, device=DEV),
                       torch.ones(64, device=DEV), torch.zeros(64, device=DEV), u.to(DEV)).tolist()
    assert set(out) == {10, 20, 40}
    for i in range(64):
        assert out[i] == plain_llama.sample(x[i], [], temperature=1.0, top_k=3, r=float(u[i])) or \
            _sampled_ok(x[i], out[i], float(u[i]), temperature=1.0, top_k=3)


def test_sample_distribution():
    """Many draws follow softmax(logits / T)."""
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0, 0.5])
    n = 20000
    u = (torch.arange(n) + 0.5) / n
    out = ops().sample(logits.repeat(n, 1).to(DEV), torch.full((n,), 0.5, device=DEV), None, None, None, u.to(DEV))
    freq = torch.bincount(out.cpu().long(), minlength=5).float() / n
    close(freq, torch.softmax(logits / 0.5, 0), 2e-4)


def test_repetition_penalty():
    g = torch.Generator().manual_seed(13)
    x = torch.randn(3, 200, generator=g)
    prev = torch.tensor([[5, 7, 5, 9, 0, 0], [1, 2, 3, 4, 5, 6], [0, 0, 0, 0, 0, 0]], dtype=torch.int32)
    n = torch.tensor([4, 6, 0], dtype=torch.int32)
    pen = torch.tensor([1.3, 2.0, 1.5])
    window = torch.tensor([0, 2, 0], dtype=torch.int32)
    ref = kernel_refs.repetition_penalty(x.clone(), prev, n, pen, window)
    out = ops().repetition_penalty(x.to(DEV), prev.to(DEV), n.to(DEV), pen.to(DEV), window.to(DEV))
    close(out, ref, 1e-6)
    # histories kept on the device: rows of a larger table in another order, one id appended by the kernel
    table = torch.zeros(5, 8, dtype=torch.int32)
    row_map = torch.tensor([3, 0, 4], dtype=torch.int32)
    table[3, :3], table[0, :5], table[4, :0] = prev[0, :3], prev[1, :5], prev[2, :0]
    pos = torch.tensor([3, 5, -1], dtype=torch.int32)
    tok = torch.tensor([int(prev[0, 3]), int(prev[1, 5]), 0], dtype=torch.int32)
    table_dev = table.to(DEV)
    out = ops().repetition_penalty(x.to(DEV), table_dev, n.to(DEV), pen.to(DEV), window.to(DEV), row_map=row_map.to(DEV),
                                   append=(pos.to(DEV), tok.to(DEV)))
    close(out, ref, 1e-6)
    assert table_dev[3, 3] == prev[0, 3] and table_dev[0, 5] == prev[1, 5]


def test_repetition_penalty_from_a_history_kept_between_steps():
    from engine_checks import penalty_history_check
    penalty_history_check(DEV)


def test_kernels_refuse_what_they_cannot_take():
    from dotllm_b200.errors import KernelError
    with pytest.raises(KernelError):
        ops().add_rmsnorm(torch.zeros(2, 8), None, torch.ones(8), 1e-5, torch.float32)     # CPU tensors
    with pytest.raises(KernelError):
        ops().linear(torch.zeros(2, 8, device=DEV), torch.zeros(4, 9, device=DEV))
    with pytest.raises(KernelError):
        ops().attention(torch.zeros(1, 3 * 1024, device=DEV), torch.zeros(1, 1, 64, 1024, device=DEV),
                        torch.zeros(1, 1, 1024, 64, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                        torch.zeros(1, dtype=torch.int32, device=DEV), torch.zeros(1, 1, dtype=torch.int32, device=DEV),
                        3, 1, 1024, 1.0)                                                    # head_dim too large


# ----------------------------------------------------------------- tensor-core kernels (bfloat16)
@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(64, 64), (200, 176), (1000, 320), (4096, 4096), (6144, 512)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_skinny(M, N, K, out_dtype, monkeypatch):
    from dotllm_b200.kernels import gemm_skinny
    monkeypatch.setattr(gemm_skinny, "SKINNY_ROWS", gemm_skinny.KERNEL_ROWS)      # every row count the kernel takes, not only those the dispatcher gives it
    g = torch.Generator().manual_seed(20)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    assert gemm_skinny.takes(x.to(DEV), w.to(DEV))
    y = gemm_skinny.run(x.to(DEV), w.to(DEV), out_dtype)
    ref = (x.double() @ w.double().T).float()
    close(y, ref, 2e-4 * math.sqrt(K / 64), 2 ** -8 if out_dtype == torch.bfloat16 else 1e-5)
    # a row's result does not depend on the other rows in the call
    y1 = gemm_skinny.run(x[:1].contiguous().to(DEV), w.to(DEV), out_dtype)
    assert torch.equal(y1.cpu(), y[:1].cpu())
    # and a second call gives the same bits (the split-k merge order is fixed, the counters are left zero)
    assert torch.equal(gemm_skinny.run(x.to(DEV), w.to(DEV), out_dtype).cpu(), y.cpu())


def test_gemm_skinny_repeats_with_full_rings(monkeypatch):
    """16 rows make the consumer warps the slower side, so the rings stay full and every slot is
    refilled the moment it is released: 30 launches must give the same bits as the first (a release
    that does not wait for the reads of the slot shows up as a few wrong output columns)."""
    from dotllm_b200.kernels import gemm_skinny
    monkeypatch.setattr(gemm_skinny, "SKINNY_ROWS", gemm_skinny.KERNEL_ROWS)
    g = torch.Generator().manual_seed(27)
    x = torch.randn(16, 4096, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(4096, 4096, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    first = gemm_skinny.run(x, w, torch.float32)
    close(first, (x.double() @ w.double().T).float(), 2e-4 * 8, 1e-5)
    for _ in range(30):
        assert torch.equal(gemm_skinny.run(x, w, torch.float32), first)


@pytest.mark.parametrize("M,H,K,N2", [(8, 4096, 512, 1024), (1, 1000, 384, 272), (13, 1000, 384, 272), (16, 72, 64, 40),
                                      (17, 1000, 384, 272), (64, 4096, 512, 1024), (100, 1000, 4096, 272), (128, 72, 64, 40)])
def test_products_that_add_and_normalise(M, H, K, N2, monkeypatch):
    """A decode step's add + RMSNorm done by the two products around it: the first adds its result
    into the float32 stream and leaves stream * gain with sums of squares per 16 columns (per 128 with more than 16 rows), the second
    multiplies its output rows by rsqrt(mean + eps).  The stream must come out with the bits of the
    separate kernels; the second product is compared with the product of the normalised rows, for a
    plain and a gated product, at widths that are no multiple of 16."""
    o = ops()
    from dotllm_b200.kernels import gemm_skinny, library
    monkeypatch.setattr(gemm_skinny, "TC_PLAIN", True)     # above 16 rows the plain products are the library's unless asked
    g = torch.Generator().manual_seed(60)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w1 = (torch.randn(H, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    w2 = (torch.randn(N2, H, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    wg = (torch.randn(2 * N2, H, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    gain = (1 + 0.3 * torch.randn(H, generator=g)).to(DEV)
    stream0 = (torch.randn(M, H, generator=g) * 2).to(DEV)
    stream0[0] *= 30                                       # rows of very different scale: a factor taken from the wrong row shows
    eps = 1e-5
    # the separate kernels
    plain_stream = stream0.clone()
    normed = o.add_rmsnorm(plain_stream, o.linear(a, w1, out_dtype=torch.float32), gain, eps, torch.bfloat16)
    # the two products
    stream = stream0.clone()
    pending = o.linear(a, w1, out_dtype=torch.float32, lazy=True)
    assert isinstance(pending, o.PendingProduct)
    rows = o.add_rmsnorm(stream, pending, gain, eps, torch.bfloat16, lazy=True)
    assert isinstance(rows, o.ScaledRows)
    assert torch.equal(stream, plain_stream)
    y = o.linear(rows, w2, out_dtype=torch.float32)
    yg = o.gated_linear(rows, wg)
    zero = torch.zeros(H, H, dtype=torch.bfloat16, device=DEV)
    chained = o.add_rmsnorm(stream, o.linear(rows, zero, out_dtype=torch.float32, lazy=True), gain, eps, torch.bfloat16,
                            lazy=True)                    # scaled rows in, stream out: both fusions in one launch
    assert isinstance(chained, o.ScaledRows) and torch.equal(stream, plain_stream)     # a zero matrix adds nothing
    stride = rows.sums.numel() // rows.row_sums()[1]      # floats between two parts of the sums
    assert torch.equal(chained.data, rows.data)
    assert torch.equal(chained.sums.view(-1, stride)[:, :M], rows.sums.view(-1, stride)[:, :M])
    library.check_status()
    # what the rows stand for
    h = plain_stream.double().cpu()
    n = h * torch.rsqrt((h * h).mean(dim=1, keepdim=True) + eps) * gain.double().cpu()
    close(rows.tensor(), n.float(), 0.0, 2 ** -8)
    assert torch.equal(rows.tensor(), normed)
    # Either way each of a row's H numbers is rounded to bfloat16 once (relative 2^-9) before the sum of
    # products, so a result is within 2^-9 sum |n_k w_k| of the exact one (plus float32 summation).
    w2d, wgd = w2.double().cpu(), wg.double().cpu()
    ref, slack = n @ w2d.T, 2 ** -9 * (n.abs() @ w2d.abs().T) * 1.05 + 1e-5
    assert bool(((y.double().cpu() - ref).abs() <= slack).all())
    gu, gu_slack = n @ wgd.T, 2 ** -9 * (n.abs() @ wgd.abs().T) * 1.05 + 1e-5
    gate, up, e_gate, e_up = gu[:, :N2], gu[:, N2:], gu_slack[:, :N2], gu_slack[:, N2:]
    want = gate * torch.sigmoid(gate) * up
    # |d silu| <= 1.1; the output is rounded to bfloat16 once more
    slack = 1.1 * e_gate * (up.abs() + e_up) + (gate * torch.sigmoid(gate)).abs() * e_up + 2 ** -8 * want.abs() + 1e-5
    assert bool(((yg.double().cpu() - want).abs() <= slack).all())
    # the same bits whatever else is in the batch: the first row alone (where the tcgen05 product runs,
    # the fewest rows that the dispatcher gives it)
    sub = 1 if M <= gemm_skinny.SKINNY_ROWS else gemm_skinny.SKINNY_ROWS + 1
    if M > sub:
        s1 = stream0[:sub].clone()
        r1 = o.add_rmsnorm(s1, o.linear(a[:sub], w1, out_dtype=torch.float32, lazy=True), gain, eps, torch.bfloat16, lazy=True)
        assert torch.equal(s1, stream[:sub]) and torch.equal(o.linear(r1, w2, out_dtype=torch.float32), y[:sub])


def test_counters_are_cleared_with_the_status_word():
    """A launch that gives up on a bounded wait may leave arrival counters counted.  ``check_status``
    raises once and clears them with the status word, so the products after the error are right
    again.  The failure is planted on the host: a status code and counters as an aborted launch
    could have left them."""
    from dotllm_b200.errors import KernelError
    from dotllm_b200.kernels import gemm_decode_tc, gemm_skinny, library
    g = torch.Generator().manual_seed(29)
    w = (torch.randn(4096, 4096, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    x = torch.randn(64, 4096, generator=g).to(torch.bfloat16).to(DEV)
    want8, want64 = gemm_skinny.run(x[:8], w, torch.float32), gemm_skinny.run(x, w, torch.float32)
    library.check_status()
    dev = torch.device("cuda", torch.cuda.current_device())
    gemm_skinny._device_state(dev)[0][:256] = 1             # as if some tiles' first parts had arrived and nothing merged them
    gemm_decode_tc._device_state(dev)[0][:32] = 1
    library.status_word(dev).fill_(3)
    with pytest.raises(KernelError):
        library.check_status()
    assert torch.equal(gemm_skinny.run(x[:8], w, torch.float32), want8)
    assert torch.equal(gemm_skinny.run(x, w, torch.float32), want64)
    library.check_status()


@pytest.mark.parametrize("M", [17, 33, 64, 65, 128])
@pytest.mark.parametrize("N,K", [(64, 64), (200, 176), (1000, 320), (4096, 4096), (6144, 512), (130, 14336)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_decode_tc(M, N, K, out_dtype):
    """The tcgen05 weight-streaming product (17 to 128 rows) against a float64 product, at sizes off its
    128 x 64 tile grid and with tiles cut between blocks (4096 x 4096: 2048 units on 148 blocks; 130 x
    14336: two tiles of 224 chunks each)."""
    from dotllm_b200.kernels import gemm_decode_tc, gemm_skinny, library
    g = torch.Generator().manual_seed(22)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    xd, wd = x.to(DEV), w.to(DEV)
    assert gemm_decode_tc.takes(xd, wd)
    y = gemm_skinny.run(xd, wd, out_dtype)                  # dispatches on the number of rows
    library.check_status()
    ref = (x.double() @ w.double().T).float()
    close(y, ref, 2e-4 * math.sqrt(K / 64), 2 ** -8 if out_dtype == torch.bfloat16 else 1e-5)
    # a row's result does not depend on the other rows in the call (17 rows: another padded width)
    y17 = gemm_decode_tc.run(xd[:17].contiguous(), wd, out_dtype)
    assert torch.equal(y17, y[:17])
    # a second call gives the same bits (the merge order of cut tiles is fixed, the counters are left zero)
    assert torch.equal(gemm_skinny.run(xd, wd, out_dtype), y)
    # rows of a wider buffer, and a product that reads its weights early
    wide = torch.zeros(M, K + 8, dtype=torch.bfloat16, device=DEV)
    wide[:, :K] = xd
    assert torch.equal(gemm_skinny.run(wide[:, :K], wd, out_dtype, resident=True), y)
    library.check_status()


@pytest.mark.parametrize("M", [17, 40, 64, 100, 128])
@pytest.mark.parametrize("I,K", [(176, 64), (512, 192), (720, 320), (14336, 256), (1000, 4096)])
def test_gemm_decode_tc_gated(M, I, K):
    from dotllm_b200.kernels import gemm_decode_tc, library
    g = torch.Generator().manual_seed(23)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, generator=g) * 0.1).to(torch.bfloat16)
    gu = x.double() @ w.double().T
    ref = plain_llama.swiglu(gu[:, :I].float(), gu[:, I:].float())
    y = gemm_decode_tc.run(x.to(DEV), w.to(DEV), torch.bfloat16, fuse_swiglu=True)
    library.check_status()
    assert y.shape == (M, I)
    close(y, ref, 2e-4 * math.sqrt(K / 64), 2 ** -8)
    assert torch.equal(gemm_decode_tc.run(x.to(DEV), w.to(DEV), torch.bfloat16, fuse_swiglu=True), y)
    assert torch.equal(ops().gated_linear(x.to(DEV), w.to(DEV)), y)


@pytest.mark.parametrize("M", [1, 8, 16])
@pytest.mark.parametrize("N,K", [(200, 176), (4096, 4096)])
def test_gemm_decode_tc_few_rows(M, N, K):
    """The tcgen05 product also takes 1 to 16 rows (padded to 16 tokens), though the dispatcher gives
    those to the mma.sync kernel."""
    from dotllm_b200.kernels import gemm_decode_tc, library
    g = torch.Generator().manual_seed(24)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    y = gemm_decode_tc.run(x.to(DEV), w.to(DEV), torch.float32)
    library.check_status()
    close(y, (x.double() @ w.double().T).float(), 2e-4 * math.sqrt(K / 64), 1e-5)


def test_gemm_decode_tc_repeats():
    """128 rows of 4096 x 4096 and 64 rows of the widest gated tile, thirty launches each: the same
    bits every time (a stage released before its MMAs have read it, or an accumulator buffer handed
    back too early, shows up as a few wrong outputs)."""
    from dotllm_b200.kernels import gemm_decode_tc, library
    g = torch.Generator().manual_seed(28)
    x = torch.randn(128, 4096, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(4096, 4096, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    first = gemm_decode_tc.run(x, w, torch.float32)
    close(first, (x.double() @ w.double().T).float(), 2e-4 * 8, 1e-5)
    for _ in range(30):
        assert torch.equal(gemm_decode_tc.run(x, w, torch.float32, resident=True), first)
    wg = (torch.randn(2 * 2048, 4096, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    first = gemm_decode_tc.run(x[:64], wg, torch.bfloat16, fuse_swiglu=True)
    for _ in range(30):
        assert torch.equal(gemm_decode_tc.run(x[:64], wg, torch.bfloat16, fuse_swiglu=True, resident=True), first)
    library.check_status()


@pytest.mark.parametrize("M,N,K", [(17, 64, 64), (128, 256, 64), (129, 257, 72), (300, 1000, 320), (2048, 384, 192),
                                   (515, 4096, 1024)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("blocks", [0, 2])
def test_gemm_tc(M, N, K, out_dtype, blocks, monkeypatch):
    """The tcgen05 product at sizes that are no multiple of its 128 x 256 x 64 tile, with all
    multiprocessors and with two blocks (many tiles per block: the stage ring wraps and both
    accumulators in tensor memory are reused)."""
    from dotllm_b200.kernels import gemm_tc, library
    monkeypatch.setattr(gemm_tc, "BLOCKS", blocks)
    g = torch.Generator().manual_seed(40)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    assert gemm_tc.takes(x.to(DEV), w.to(DEV))
    y = gemm_tc.run(x.to(DEV), w.to(DEV), out_dtype)
    library.check_status()
    ref = (x.double() @ w.double().T).float()
    close(y, ref, 2e-4 * math.sqrt(K / 64), 2 ** -8 if out_dtype == torch.bfloat16 else 1e-5)
    assert torch.equal(gemm_tc.run(x.to(DEV), w.to(DEV), out_dtype).cpu(), y.cpu())
    # rows of a wider buffer (a row stride larger than K)
    wide = torch.zeros(M, K + 8, dtype=torch.bfloat16, device=DEV)
    wide[:, :K] = x.to(DEV)
    assert torch.equal(gemm_tc.run(wide[:, :K], w.to(DEV), out_dtype).cpu(), y.cpu())


@pytest.mark.parametrize("M,I,K", [(40, 176, 64), (300, 720, 320), (2048, 1024, 256), (130, 14336, 128)])
@pytest.mark.parametrize("blocks", [0, 3])
def test_gemm_tc_gated(M, I, K, blocks, monkeypatch):
    from dotllm_b200.kernels import gemm_tc, library
    monkeypatch.setattr(gemm_tc, "BLOCKS", blocks)
    g = torch.Generator().manual_seed(41)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, generator=g) * 0.1).to(torch.bfloat16)
    gu = x.double() @ w.double().T
    ref = plain_llama.swiglu(gu[:, :I].float(), gu[:, I:].float())
    y = gemm_tc.run(x.to(DEV), w.to(DEV), torch.bfloat16, fuse_swiglu=True)
    library.check_status()
    assert y.shape == (M, I)
    close(y, ref, 2e-4, 2 ** -8)


@pytest.mark.parametrize("M", [1, 5, 16, 40])
@pytest.mark.parametrize("I,K", [(176, 64), (512, 192), (720, 320), (14336, 256)])
def test_gemm_skinny_gated(M, I, K):
    from dotllm_b200.kernels import gemm_skinny
    g = torch.Generator().manual_seed(21)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, generator=g) * 0.1).to(torch.bfloat16)
    gu = x.double() @ w.double().T
    ref = plain_llama.swiglu(gu[:, :I].float(), gu[:, I:].float())
    if M <= gemm_skinny.MAX_ROWS:
        y = gemm_skinny.run(x.to(DEV), w.to(DEV), torch.bfloat16, fuse_swiglu=True)
        assert y.shape == (M, I)
        close(y, ref, 2e-4, 2 ** -8)
    # the op picks the fused kernel for few rows and the two-kernel path otherwise; both agree
    # The two-kernel path rounds gate and up to bfloat16 (relative step 2^-8) before the gating:
    # |d silu(g)u| <= 2^-8 (|g silu'(g) u| + |silu(g) u|), plus the output's own rounding.
    both = ops().gated_linear(x.to(DEV), w.to(DEV))
    gate, up = gu[:, :I].float(), gu[:, I:].float()
    sig = torch.sigmoid(gate)
    dsilu = sig * (1 + gate * (1 - sig))
    bound = 2 ** -8 * ((gate * dsilu * up).abs() + 2 * ref.abs()) + 2e-4
    assert bool(((both.float().cpu() - ref).abs() <= bound).all())


def _decode_plan(lengths):
    from dotllm_b200.engine.step import AttentionPlan
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    n = len(lengths)
    return AttentionPlan(n_seqs=n, max_new=1, max_total=max(lengths), all_single=True,
                         seq_start=t([v - 1 for v in lengths]), seq_new=t([1] * n), cu_new=t(list(range(n + 1))),
                         seq_total=t(lengths), starts=[v - 1 for v in lengths], news=[1] * n)


@pytest.mark.parametrize("nh,nkv,hd", [(6, 6, 32), (8, 2, 64), (32, 8, 128), (16, 1, 128), (12, 4, 96), (3, 1, 64)])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("blocks", [0, 7, 1])
def test_attention_decode_split_keys(nh, nkv, hd, window, blocks, monkeypatch):
    """One token per sequence, lengths from 1 to many pages of keys, pages scattered, NaN in every
    place that no live key holds.  The step's pages are cut into equal shares for every
    multiprocessor, for 7 blocks (shares that hold whole sequences between two cut ones) and for
    one block (nothing cut)."""
    from dotllm_b200.kernels import attention_fast
    monkeypatch.setattr(attention_fast, "DECODE_BLOCKS", blocks)
    lengths = [1, 31, 32, 33, 64, 65, 255, 256, 257, 700, 1500]
    k_pool, v_pool, table, dense = make_paged(len(lengths), lengths, nkv, hd, torch.bfloat16, seed=22)
    g = torch.Generator().manual_seed(23)
    q = torch.randn(len(lengths), nh * hd, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(hd)
    seqs = torch.arange(len(lengths), dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    args = (q.to(DEV), k_pool.to(DEV), v_pool.to(DEV), seqs, pos, table.to(DEV), nh, nkv, hd, scale, window)
    fast = ops().attention(*args, plan=_decode_plan(lengths))
    generic = ops().attention(*args)
    ref = torch.stack([dense_attention(q[b], *dense[b], nh, nkv, scale, lengths[b] - 1, window)
                       for b in range(len(lengths))])
    assert bool(torch.isfinite(fast).all())
    close(fast, ref, 2e-3, 2 ** -7)
    close(generic, ref, 2e-3, 2 ** -7)
    again = ops().attention(*args, plan=_decode_plan(lengths))
    assert torch.equal(fast.cpu(), again.cpu())


@pytest.mark.parametrize("nh,nkv,hd,rotate", [(8, 2, 64, True), (32, 8, 128, True), (16, 1, 128, True), (6, 6, 32, False),
                                              (12, 4, 96, False), (8, 2, 128, False)])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("blocks", [0, 5])
def test_attention_decode_with_the_new_token_inside(nh, nkv, hd, rotate, window, blocks, monkeypatch):
    """A decode step as one kernel (rotation of q and k, cache write, attention) against the same
    step as two kernels: the same output bits and the same cache contents.  The new token lands at
    the start, in the middle and at the end of a page."""
    from dotllm_b200.kernels import attention_fast, library
    monkeypatch.setattr(attention_fast, "DECODE_BLOCKS", blocks)
    lengths = [1, 64, 65, 128, 200, 700, 1500, 33]
    B = len(lengths)
    k_pool, v_pool, table, _ = make_paged(B, lengths, nkv, hd, torch.bfloat16, seed=60)
    g = torch.Generator().manual_seed(61)
    qkv = torch.randn(B, (nh + 2 * nkv) * hd, generator=g).to(torch.bfloat16)
    cos, sin = plain_llama.rope_tables(range(2048), hd, 10000.0) if rotate else (None, None)
    rd = hd if rotate else 0
    seqs = torch.arange(B, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    d = lambda t: None if t is None else t.to(DEV)

    def run(fused):
        x = qkv.to(DEV).clone()
        q, k, v = x[:, :nh * hd], x[:, nh * hd:(nh + nkv) * hd], x[:, (nh + nkv) * hd:]
        kp, vp = k_pool.to(DEV).clone(), v_pool.to(DEV).clone()
        args = (q, k, v, d(cos), d(sin), rd, seqs, pos, table.to(DEV), kp, vp, nh, nkv, hd, 1.0 / math.sqrt(hd), window)
        if fused:
            out = ops().rope_cache_attention(*args, plan=_decode_plan(lengths))
        else:
            ops().rope_cache_write(*args[:14])
            out = ops().attention(q, kp, vp, seqs, pos, table.to(DEV), nh, nkv, hd, 1.0 / math.sqrt(hd), window,
                                  plan=_decode_plan(lengths))
        library.check_status()
        live = torch.stack([kp[int(table[b, (n - 1) // 64]), :, (n - 1) % 64] for b, n in enumerate(lengths)])
        live_v = torch.stack([vp[int(table[b, (n - 1) // 64]), :, :, (n - 1) % 64] for b, n in enumerate(lengths)])
        return out, live, live_v

    calls = []
    real = library.call
    monkeypatch.setattr(library, "call", lambda name, *a: (calls.append(name), real(name, *a))[1])
    one, k_one, v_one = run(True)
    assert calls == ["dl_attention_decode_fresh_bf16"], calls            # really one kernel
    two, k_two, v_two = run(False)
    assert bool(torch.isfinite(one).all())
    assert torch.equal(one, two)
    assert torch.equal(k_one, k_two) and torch.equal(v_one, v_two)


@pytest.mark.parametrize("fused", [False, True])
def test_attention_decode_rows_that_hold_nothing(fused):
    """Rows whose length after the step is 0 (the idle rows of a captured step wider than its batch)
    get no work: the live rows come out with the same bits as without them, and the page the idle
    rows point to is left as it was."""
    from dotllm_b200.kernels import library
    nh, nkv, hd = 8, 2, 64
    live_lengths = [70, 200, 1, 640]
    k_pool, v_pool, table, _ = make_paged(4, live_lengths, nkv, hd, torch.bfloat16, seed=70, n_pages=30)
    used = set(table[table >= 0].tolist())
    idle_page = [p for p in range(30) if p not in used][0]
    k_pool[idle_page], v_pool[idle_page] = 3.0, 5.0
    rows = [None, 0, None, None, 1, 2, None, 3, None]                  # None: idle
    B = len(rows)
    g = torch.Generator().manual_seed(71)
    qkv_live = torch.randn(4, (nh + 2 * nkv) * hd, generator=g).to(torch.bfloat16)
    cos, sin = plain_llama.rope_tables(range(1024), hd, 10000.0)
    scale = 1.0 / math.sqrt(hd)

    def run(with_idle):
        if with_idle:
            lengths = [0 if r is None else live_lengths[r] for r in rows]
            qkv = torch.stack([torch.full_like(qkv_live[0], 7.0) if r is None else qkv_live[r] for r in rows])
            tab = torch.full((B, table.shape[1]), -1, dtype=torch.int32)
            for i, r in enumerate(rows):
                if r is None:
                    tab[i, 0] = idle_page
                else:
                    tab[i] = table[r]
        else:
            lengths, qkv, tab = live_lengths, qkv_live, table
        n = len(lengths)
        x = qkv.to(DEV).clone()
        q, k, v = x[:, :nh * hd], x[:, nh * hd:(nh + nkv) * hd], x[:, (nh + nkv) * hd:]
        kp, vp = k_pool.to(DEV).clone(), v_pool.to(DEV).clone()
        seqs = torch.arange(n, dtype=torch.int32, device=DEV)
        pos = torch.tensor([max(0, v - 1) for v in lengths], dtype=torch.int32, device=DEV)
        plan = _decode_plan(lengths)
        plan.seq_start = pos
        if fused:
            out = ops().rope_cache_attention(q, k, v, cos.to(DEV), sin.to(DEV), hd, seqs, pos, tab.to(DEV), kp, vp,
                                             nh, nkv, hd, scale, 0, plan=plan)
        else:
            live = torch.tensor([i for i, v in enumerate(lengths) if v > 0], dtype=torch.long, device=DEV)
            ql, kl, vl = q[live].contiguous(), k[live].contiguous(), v[live].contiguous()
            ops().rope_cache_write(ql, kl, vl, cos.to(DEV), sin.to(DEV), hd, seqs[:len(live)].contiguous(),
                                   pos[live].contiguous(), tab.to(DEV)[live].contiguous(), kp, vp, nh, nkv, hd)
            q = q.clone()
            q[live] = ql
            out = ops().attention(q, kp, vp, seqs, pos, tab.to(DEV), nh, nkv, hd, scale, 0, plan=plan)
        library.check_status()
        return out, kp, vp

    alone, k_alone, v_alone = run(False)
    padded, k_padded, v_padded = run(True)
    keep = [i for i, r in enumerate(rows) if r is not None]
    assert bool(torch.isfinite(alone).all())
    assert torch.equal(padded[keep], alone)
    bits = lambda t: t.view(torch.int16)                               # unused places hold NaN
    assert torch.equal(bits(k_padded), bits(k_alone)) and torch.equal(bits(v_padded), bits(v_alone))
    assert bool((k_padded[idle_page] == 3.0).all()) and bool((v_padded[idle_page] == 5.0).all())


def test_attention_decode_far_key():
    nh, nkv, hd, n = 8, 2, 128, 3000
    k_pool, v_pool, table, dense = make_paged(1, [n], nkv, hd, torch.bfloat16, seed=24)
    k, v = dense[0]
    q = torch.zeros(1, nh * hd)
    far = 70
    for h in range(nh):
        q[0, h * hd:(h + 1) * hd] = k[far, h // 4] * 8.0
    out = ops().attention(q.to(torch.bfloat16).to(DEV), k_pool.to(DEV), v_pool.to(DEV),
                          torch.zeros(1, dtype=torch.int32, device=DEV), torch.tensor([n - 1], dtype=torch.int32, device=DEV),
                          table.to(DEV), nh, nkv, hd, 1 / math.sqrt(hd), 0, plan=_decode_plan([n]))
    want = torch.cat([v[far, h // 4] for h in range(nh)])
    close(out[0], want, 2e-2)


def _prefill_plan(lengths, news):
    from dotllm_b200.engine.step import AttentionPlan
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    starts = [n - m for n, m in zip(lengths, news)]
    cu = [0]
    for m in news:
        cu.append(cu[-1] + m)
    return AttentionPlan(n_seqs=len(lengths), max_new=max(news), max_total=max(lengths),
                         all_single=all(m == 1 for m in news), seq_start=t(starts), seq_new=t(news), cu_new=t(cu),
                         seq_total=t(lengths), starts=starts, news=list(news))


@pytest.mark.parametrize("nh,nkv,hd", [(6, 6, 32), (8, 2, 64), (8, 2, 128), (5, 1, 96)])
@pytest.mark.parametrize("window", [0, 90])
@pytest.mark.parametrize("tc", [True, False])
def test_attention_prefill_packed_unequal(nh, nkv, hd, window, tc, monkeypatch):
    """Whole prompts, a chunk appended to earlier context, and single tokens in one packed call:
    by the tcgen05 kernel (head sizes 64 and 128) and by the mma.sync kernel (every size)."""
    from dotllm_b200.kernels import attention_fast
    monkeypatch.setattr(attention_fast, "PREFILL_TC", tc)
    _check_prefill_packed(nh, nkv, hd, window, lengths=[1, 70, 333, 64, 500, 129], news=[1, 70, 33, 1, 500, 65])


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("window", [0, 40, 200])
def test_attention_prefill_tc_tile_edges(hd, window):
    """The tcgen05 kernel takes 256 rows a block as two tiles of 128 that share their pages: prompts
    that end exactly at a tile's or a block's edge or one row past it, alone and behind earlier
    context of odd length, and windows shorter and longer than a tile (with a short window the
    second tile joins the walk pages after the first)."""
    _check_prefill_packed(4, 2, hd, window, lengths=[128, 134, 256 + 64, 257 + 100, 385, 511 + 7],
                          news=[128, 129, 256, 257, 385, 511])


def _check_prefill_packed(nh, nkv, hd, window, lengths, news):
    k_pool, v_pool, table, dense = make_paged(len(lengths), lengths, nkv, hd, torch.bfloat16, seed=30)
    g = torch.Generator().manual_seed(31)
    token_seq, token_pos = [], []
    for b, (n, new) in enumerate(zip(lengths, news)):
        for p in range(n - new, n):
            token_seq.append(b)
            token_pos.append(p)
    T = len(token_seq)
    q = torch.randn(T, nh * hd, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(hd)
    args = (q.to(DEV), k_pool.to(DEV), v_pool.to(DEV), torch.tensor(token_seq, dtype=torch.int32, device=DEV),
            torch.tensor(token_pos, dtype=torch.int32, device=DEV), table.to(DEV), nh, nkv, hd, scale, window)
    fast = ops().attention(*args, plan=_prefill_plan(lengths, news))
    ref = torch.stack([dense_attention(q[t], *dense[token_seq[t]], nh, nkv, scale, token_pos[t], window)
                       for t in range(T)])
    assert bool(torch.isfinite(fast).all())
    # The tensor-core kernel rounds the softmax weights to bfloat16 (relative step 2^-9 after
    # rounding to nearest) for the P V product: |error| <= 2^-9 max|v|, plus the output's rounding.
    v_max = max(float(v.abs().max()) for _, v in dense)
    close(fast, ref, 2 ** -9 * v_max + 1e-3, 2 ** -8)
    from dotllm_b200.kernels import library
    library.check_status()


@pytest.mark.parametrize("hd,window", [(128, 0), (64, 0), (128, 700)])
def test_attention_prefill_tc_long_prompt(hd, window):
    """A prompt of 40 pages appended to 3 pages of context: the stage ring of the tcgen05 kernel
    wraps many times, both score buffers and both weight buffers are reused, and one far key per
    head carries a large score, so that a lost page or a wrong rescale of the running output shows.
    Compared with the generic kernel (one warp per token and head, float32 softmax)."""
    from dotllm_b200.kernels import library
    nh, nkv = 4, 2
    start, new = 170, 2500
    lengths, news = [start + new], [new]
    k_pool, v_pool, table, dense = make_paged(1, lengths, nkv, hd, torch.bfloat16, seed=33)
    g = torch.Generator().manual_seed(34)
    q = torch.randn(new, nh * hd, generator=g).to(torch.bfloat16)
    # rows from position 2000 on look for key 1234 of their KV head (unless the window hides it)
    k_dense = dense[0][0]
    for h in range(nh):
        q[2000 - start:, h * hd:(h + 1) * hd] = (k_dense[1234, h // (nh // nkv)].float() * 3.0).to(torch.bfloat16)
    token_seq = torch.zeros(new, dtype=torch.int32, device=DEV)
    token_pos = torch.arange(start, start + new, dtype=torch.int32, device=DEV)
    args = (q.to(DEV), k_pool.to(DEV), v_pool.to(DEV), token_seq, token_pos, table.to(DEV), nh, nkv, hd,
            1.0 / math.sqrt(hd), window)
    fast = ops().attention(*args, plan=_prefill_plan(lengths, news))
    library.check_status()
    generic = ops().attention(*args)
    assert bool(torch.isfinite(fast).all())
    v_max = float(dense[0][1].abs().max())
    close(fast, generic, 2 ** -9 * v_max + 2e-3, 2 ** -7)


@pytest.mark.parametrize("blocks", [0, 3])
def test_attention_decode_long_runs(monkeypatch, blocks):
    """Few sequences and long caches: a (sequence, head) is spread over tens of blocks, or, with
    three blocks, every warp takes hundreds of pages and the ring of stages wraps many times."""
    from dotllm_b200.kernels import attention_fast
    monkeypatch.setattr(attention_fast, "DECODE_BLOCKS", blocks)
    nh, nkv, hd = 32, 8, 128
    lengths = [8192, 5001, 64]
    k_pool, v_pool, table, dense = make_paged(len(lengths), lengths, nkv, hd, torch.bfloat16, seed=25)
    q = torch.randn(len(lengths), nh * hd, generator=torch.Generator().manual_seed(26)).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(hd)
    seqs = torch.arange(len(lengths), dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    args = (q.to(DEV), k_pool.to(DEV), v_pool.to(DEV), seqs, pos, table.to(DEV), nh, nkv, hd, scale, 0)
    fast = ops().attention(*args, plan=_decode_plan(lengths))
    generic = ops().attention(*args)
    assert bool(torch.isfinite(fast).all())
    v_max = max(float(v.abs().max()) for _, v in dense)
    close(fast, generic, 2 ** -9 * v_max + 1e-3, 2 ** -7)
    from dotllm_b200.kernels import library
    library.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_score_hook(dtype):
    """Scores capped by softcap * tanh(s / softcap) and biased by a slope per head times the distance,
    on the generic kernel (the tensor-core kernels take no hook: with one the op must not use them)."""
    o = ops()
    nh, nkv, hd = 4, 2, 32
    lengths = [70, 5, 130]
    k_pool, v_pool, table, _ = make_paged(3, lengths, nkv, hd, dtype, seed=31)
    g = torch.Generator().manual_seed(32)
    q = (torch.randn(3, nh * hd, generator=g) * 2).to(dtype)
    seqs = torch.arange(3, dtype=torch.int32)
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32)
    slopes = torch.tensor([0.3, 0.0, 0.02, 1.0])
    hook = o.ScoreHook(softcap=2.5, slopes=slopes.to(DEV))
    plan = _decode_plan(lengths)                              # a plan is at hand: the hook alone keeps the fast kernels out
    got = o.attention(q.to(DEV), k_pool.to(DEV), v_pool.to(DEV), seqs.to(DEV), pos.to(DEV), table.to(DEV), nh, nkv, hd,
                      0.2, 0, plan=plan, score_hook=hook)
    want = kernel_refs.attention(q, k_pool, v_pool, seqs, pos, table, nh, nkv, hd, 0.2, 0,
                                 score_hook=o.ScoreHook(2.5, slopes))
    close(got, want, 2e-5 if dtype == torch.float32 else 2e-2, 0.0)
    plain = o.attention(q.to(DEV), k_pool.to(DEV), v_pool.to(DEV), seqs.to(DEV), pos.to(DEV), table.to(DEV), nh, nkv, hd, 0.2, 0)
    assert float((plain.float() - got.float()).abs().max()) > 1e-2     # the hook does change the result
