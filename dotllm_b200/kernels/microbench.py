"""Time one kernel alone at a given size (CUDA events, warm-up, L2 flushed between runs).

    python -m dotllm_b200.kernels.microbench attention_decode --batch 8 --context 8192
    python -m dotllm_b200.kernels.microbench gemm_skinny --rows 8 --n 28672 --k 4096 --gated
    python -m dotllm_b200.kernels.microbench attention_prefill --tokens 2048
    python -m dotllm_b200.kernels.microbench norm --rows 8 --width 4096
    python -m dotllm_b200.kernels.microbench rope --rows 8
    python -m dotllm_b200.kernels.microbench sample --rows 8 --top-k 40 --top-p 0.95

Prints one JSON line with the time, the algorithmic bytes or FLOPs, and the fraction of the
measured peak.  The same command under ``ncu -k regex:<kernel>`` gives the kernel's counters.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        d = json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except (OSError, ValueError, KeyError):
        return 6650.0, 1590.0, "fallback"


def _time(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.add_(1)                                   # more bytes than the L2 holds
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2], times[0]


def _time_graph(fn, iters):
    """Median time of one replay of ``fn`` captured as a CUDA graph."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2]


SCATTER_PAGES = True       # pages of a sequence in random order (False: in the order they were taken)


def _paged(batch, context, nkv, hd, dev):
    pages_per = (context + 63) // 64
    n_pages = batch * pages_per
    k_pool = torch.randn(n_pages, nkv, 64, hd, device=dev, dtype=torch.bfloat16)
    v_pool = torch.randn(n_pages, nkv, hd, 64, device=dev, dtype=torch.bfloat16)
    order = torch.randperm(n_pages, device=dev) if SCATTER_PAGES else torch.arange(n_pages, device=dev)
    table = order.to(torch.int32).view(batch, pages_per).contiguous()
    return k_pool, v_pool, table


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["attention_decode", "attention_prefill", "gemm_skinny", "gemm_tc", "norm", "rope", "sample"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--width", type=int, default=4096)
    ap.add_argument("--gated", action="store_true")
    ap.add_argument("--skinny-rows", type=int, default=None,
                    help="gemm_skinny: most rows that go to the mma.sync kernel (more go to the tcgen05 one)")
    ap.add_argument("--out-f32", action="store_true")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--decode-blocks", type=int, default=0, help="attention_decode: persistent blocks (0: one per multiprocessor)")
    ap.add_argument("--timeline", action="store_true",
                    help="attention_prefill: print the per-page timeline of the tcgen05 kernel (needs a library built "
                         "with DOTLLM_NVCC_EXTRA=-DPT_TIMELINE)")
    ap.add_argument("--no-tc", action="store_true", help="attention_prefill: the mma.sync kernel instead of the tcgen05 one")
    ap.add_argument("--sequential-pages", action="store_true", help="pages of a sequence lie one after another")
    ap.add_argument("--vocab", type=int, default=128256, help="sample: entries of a row of logits")
    ap.add_argument("--top-k", type=int, default=0, help="sample: top-k (0: off)")
    ap.add_argument("--top-p", type=float, default=1.0, help="sample: top-p (1: off)")
    ap.add_argument("--one-block", action="store_true", help="sample: one block per row instead of a cluster of blocks")
    args = ap.parse_args(argv)
    if args.sequential_pages:
        global SCATTER_PAGES
        SCATTER_PAGES = False

    from ..engine.step import AttentionPlan
    from . import gemm_skinny, ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hbm, tflops, source = _peaks()
    flush = None if args.no_flush else torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    nh, nkv, hd = args.heads, args.kv_heads, args.head_dim
    t32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    result = {"kernel": args.kernel}

    if args.kernel == "attention_decode":
        if args.decode_blocks:
            from . import attention_fast
            attention_fast.DECODE_BLOCKS = args.decode_blocks
        b, ctx = args.batch, args.context
        k_pool, v_pool, table = _paged(b, ctx, nkv, hd, dev)
        q = torch.randn(b, nh * hd, device=dev, dtype=torch.bfloat16)
        plan = AttentionPlan(n_seqs=b, max_new=1, max_total=ctx, all_single=True, seq_start=t32([ctx - 1] * b),
                             seq_new=t32([1] * b), cu_new=t32(list(range(b + 1))), seq_total=t32([ctx] * b),
                             starts=[ctx - 1] * b, news=[1] * b)
        seqs, pos = t32(list(range(b))), t32([ctx - 1] * b)
        fn = lambda: ops.attention(q, k_pool, v_pool, seqs, pos, table, nh, nkv, hd, 1 / math.sqrt(hd), 0, plan=plan)
        nbytes = 2 * b * ctx * nkv * hd * 2
        ms, best = _time(fn, args.iters, flush)
        result.update(batch=b, context=ctx, bytes=nbytes, ms=ms, best_ms=best, gbs=nbytes / ms / 1e6,
                      frac_of_hbm=nbytes / ms / 1e6 / hbm)
        # As a decode step issues it: launches back to back from a captured graph (no host in the
        # timed region), each on its own cache (together larger than the L2).
        copies = max(2, (300 << 20) // nbytes + 1)
        caches = [(k_pool, v_pool, table)] + [_paged(b, ctx, nkv, hd, dev) for _ in range(copies - 1)]
        chained = _time_graph(lambda: [ops.attention(q, kp, vp, seqs, pos, tb, nh, nkv, hd, 1 / math.sqrt(hd), 0, plan=plan)
                                       for kp, vp, tb in caches], args.iters) / copies
        result.update(chained_ms=chained, chained_gbs=nbytes / chained / 1e6, chained_frac_of_hbm=nbytes / chained / 1e6 / hbm)
    elif args.kernel == "attention_prefill":
        if args.no_tc:
            from . import attention_fast
            attention_fast.PREFILL_TC = False
        T = args.tokens
        k_pool, v_pool, table = _paged(1, T, nkv, hd, dev)
        q = torch.randn(T, nh * hd, device=dev, dtype=torch.bfloat16)
        plan = AttentionPlan(n_seqs=1, max_new=T, max_total=T, all_single=False, seq_start=t32([0]), seq_new=t32([T]),
                             cu_new=t32([0, T]), seq_total=t32([T]), starts=[0], news=[T])
        seqs, pos = t32([0] * T), t32(list(range(T)))
        fn = lambda: ops.attention(q, k_pool, v_pool, seqs, pos, table, nh, nkv, hd, 1 / math.sqrt(hd), 0, plan=plan)
        flops = 2 * T * T * nh * hd                        # causal: half of 4 T^2 nh hd
        ms, best = _time(fn, args.iters, flush)
        if args.timeline:
            import ctypes
            from . import library
            lib = library.library()
            if not hasattr(lib, "dl_attention_prefill_tc_timeline"):
                raise SystemExit("the library was not built with DOTLLM_NVCC_EXTRA=-DPT_TIMELINE")
            pages = 256
            buf = (ctypes.c_longlong * (12 * pages))()
            lib.dl_attention_prefill_tc_timeline.argtypes = [ctypes.c_void_p]
            if lib.dl_attention_prefill_tc_timeline(buf) != 0:
                raise SystemExit("could not read the timeline")
            at = lambda r, j: buf[r * pages + j]
            lo, hi = 40, min(100, (T + 63) // 64 - 2)        # steady state, away from the diagonal's mask
            mean = lambda a, b: sum(at(b, j) - at(a, j) for j in range(lo, hi)) / (hi - lo)
            result["timeline_cycles"] = {
                "page_period": (at(0, hi) - at(0, lo)) / (hi - lo),
                "issue_scores": mean(0, 1), "wait_weights": mean(2, 3), "issue_product": mean(3, 4),
                "softmax_wait_scores": mean(5, 6), "softmax_read_scores": mean(6, 7), "softmax_maximum": mean(7, 8),
                "softmax_wait_weights_buffer": mean(8, 10), "softmax_exponentials_and_store": mean(10, 11),
                "softmax_fence_and_announce": mean(11, 9)}
        result.update(tokens=T, flops=flops, ms=ms, best_ms=best, tflops=flops / ms / 1e9,
                      frac_of_bf16_peak=flops / ms / 1e9 / tflops)
    elif args.kernel == "gemm_skinny":
        M, N, K = args.rows, args.n, args.k
        if args.skinny_rows is not None:
            gemm_skinny.SKINNY_ROWS = args.skinny_rows
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn((2 if args.gated else 1) * N, K, device=dev, dtype=torch.bfloat16) * 0.02
        out_dtype = torch.float32 if args.out_f32 else torch.bfloat16
        fn = lambda: gemm_skinny.run(x, w, out_dtype, fuse_swiglu=args.gated)
        nbytes = w.numel() * 2
        ms, best = _time(fn, args.iters, flush)
        result.update(rows=M, n=N, k=K, gated=args.gated, bytes=nbytes, ms=ms, best_ms=best, gbs=nbytes / ms / 1e6,
                      frac_of_hbm=nbytes / ms / 1e6 / hbm)
        lib_fn = lambda: torch.mm(x, w.t())
        lib_ms, _ = _time(lib_fn, args.iters, flush)
        result["library_mm_ms"] = lib_ms
        if args.timeline:
            import ctypes
            from . import library
            lib = library.library()
            if not hasattr(lib, "dl_gemm_skinny_timeline"):
                raise SystemExit("the library was not built with DOTLLM_NVCC_EXTRA=-DGS_TIMELINE")
            flush.add_(1)
            torch.cuda.synchronize()
            fn()                                            # one cold launch
            torch.cuda.synchronize()
            buf = (ctypes.c_longlong * (6 * 2048))()
            lib.dl_gemm_skinny_timeline.argtypes = [ctypes.c_void_p]
            if lib.dl_gemm_skinny_timeline(buf) != 0:
                raise SystemExit("could not read the timeline")
            stride = 8                                      # warps of a block: six consumers, the producer, the statistics warp
            blocks = min(148, 2048 // stride)
            first = min(buf[b * stride] for b in range(blocks) if buf[b * stride])
            names = ["block_start", "barriers_ready", "first_chunk_landed", "last_chunk_consumed", "share_done", "block_end"]
            spread = {}
            for e, name in enumerate(names):
                warps = [0] if e in (0, 1, 5) else range(6)
                v = [buf[e * 2048 + b * stride + w] - first for b in range(blocks) for w in warps
                     if buf[e * 2048 + b * stride + w]]
                spread[name] = [min(v), sum(v) // len(v), max(v)]
            result["timeline_ns_min_mean_max"] = spread
        # The same product as a decode step issues it: launches back to back from a captured graph,
        # each on a different copy of W (together larger than the L2), with and without the
        # overlap of programmatic dependent launch.
        copies = max(2, (300 << 20) // nbytes + 1)
        ws = [w] + [w.clone() for _ in range(copies - 1)]
        from . import library
        for name, dependent in (("chained_ms", True), ("chained_serial_ms", False)):
            library.set_dependent_launch(dependent)
            result[name] = _time_graph(lambda: [gemm_skinny.run(x, wi, out_dtype, fuse_swiglu=args.gated, resident=True)
                                                for wi in ws], args.iters) / copies
        library.set_dependent_launch(True)
        result["chained_gbs"] = nbytes / result["chained_ms"] / 1e6
    elif args.kernel == "gemm_tc":
        from . import gemm_tc
        M, N, K = args.rows, args.n, args.k
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn((2 if args.gated else 1) * N, K, device=dev, dtype=torch.bfloat16) * 0.02
        out_dtype = torch.float32 if args.out_f32 else torch.bfloat16
        fn = lambda: gemm_tc.run(x, w, out_dtype, fuse_swiglu=args.gated)
        flops = 2 * M * w.shape[0] * K
        ms, best = _time(fn, args.iters, flush)
        result.update(rows=M, n=N, k=K, gated=args.gated, flops=flops, ms=ms, best_ms=best, tflops=flops / ms / 1e9,
                      frac_of_bf16_peak=flops / ms / 1e9 / tflops)
        if args.gated:
            lib_fn = lambda: ops.swiglu(torch.mm(x, w.t()))
        else:
            lib_fn = lambda: torch.mm(x, w.t()) if out_dtype == torch.bfloat16 else torch.mm(x, w.t(), out_dtype=out_dtype)
        lib_ms, _ = _time(lib_fn, args.iters, flush)
        result.update(library_ms=lib_ms, library_tflops=flops / lib_ms / 1e9)
    elif args.kernel == "norm":
        rows, width = args.rows, args.width
        res = torch.randn(rows, width, device=dev)
        delta = torch.randn(rows, width, device=dev)
        gain = torch.ones(width, device=dev)
        fn = lambda: ops.add_rmsnorm(res, delta, gain, 1e-5, torch.bfloat16)
        ms, best = _time(fn, args.iters, flush)
        result.update(rows=rows, width=width, ms=ms, best_ms=best)
    elif args.kernel == "rope":
        rows = args.rows
        qkv = torch.randn(rows, (nh + 2 * nkv) * hd, device=dev, dtype=torch.bfloat16)
        if rows <= 64:                                      # a decode step: one token of each of `rows` sequences
            k_pool, v_pool, table = _paged(rows, 128, nkv, hd, dev)
            cos = torch.rand(256, hd // 2, device=dev)
            sin = torch.rand(256, hd // 2, device=dev)
            seqs, pos = t32(list(range(rows))), t32([100] * rows)
        else:                                               # a prompt: `rows` tokens of one sequence
            k_pool, v_pool, table = _paged(1, (rows + 63) // 64, nkv, hd, dev)
            cos = torch.rand(rows, hd // 2, device=dev)
            sin = torch.rand(rows, hd // 2, device=dev)
            seqs, pos = t32([0] * rows), t32(list(range(rows)))
            result["bytes"] = qkv.numel() * 2 + nh * hd * rows * 2 + 2 * nkv * hd * rows * 2
        qd, kvd = nh * hd, nkv * hd
        fn = lambda: ops.rope_cache_write(qkv[:, :qd], qkv[:, qd:qd + kvd], qkv[:, qd + kvd:], cos, sin, hd, seqs, pos,
                                          table, k_pool, v_pool, nh, nkv, hd)
        ms, best = _time(fn, args.iters, flush)
        result.update(rows=rows, ms=ms, best_ms=best)
    elif args.kernel == "sample":
        # a temperature draw (optionally top-k and top-p) for `rows` rows of `vocab` logits; 20 launches a graph
        rows, vocab = args.rows, args.vocab
        x = torch.randn(rows, vocab, device=dev) * 3
        one, u = torch.ones(rows, device=dev), torch.rand(rows, device=dev)
        kw = {}
        if args.top_k:
            kw["top_k"] = torch.full((rows,), args.top_k, dtype=torch.int32, device=dev)
        if args.top_p < 1.0:
            kw["top_p"] = one * args.top_p
        fn = lambda: ops.sample(x, temperature=one * 0.8, uniform=u, split=not args.one_block, **kw)
        ms = _time_graph(lambda: [fn() for _ in range(20)], args.iters) / 20
        result.update(rows=rows, vocab=vocab, top_k=args.top_k, top_p=args.top_p, one_block=args.one_block, ms=ms,
                      bytes=rows * vocab * 4)
    result["peaks"] = source
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
