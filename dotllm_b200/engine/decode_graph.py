"""Decode steps replayed as CUDA graphs.

A decode step launches a few hundred small kernels; issued one by one the host cannot keep up
with the device (the reference pays ~14 launches per layer per token,
src/DotLLM.Cuda/CudaTransformerModel.cs:198-286).  Here the whole forward pass of a step that
brings one token per sequence is captured once per batch size (or once per width, for the batch
sizes up to it, with idle rows: the generation loop's way) and replayed.  Everything that
changes from step to step - tokens, positions, lengths, slots, block tables - lives in fixed device
buffers that one pinned host-to-device copy refreshes before each replay, so a captured graph
serves any set of sequences of its batch size, wherever they are in the cache.

The same kernels run, on the same data, as in an eager step: graphs change launch cost only.
"""
from __future__ import annotations

import time
import warnings

import numpy as np
import torch

from ..cache.model_cache import PAGE
from ..errors import StepError
from .step import AttentionPlan, StepContext

_RING = 4            # pinned staging buffers in flight


class _Captured:
    def __init__(self, model, cache, batch, pages, n_groups):
        dev = model.runtime.device
        self.batch, self.pages = batch, pages
        self.idle_slot, self.idle_pages = cache.idle_slot, [cache.idle_page]
        self.capacity = pages * PAGE                       # longest sequence this graph serves
        n = 3 * batch + n_groups * batch * pages           # positions, lengths, slots, block tables
        self.ints = torch.zeros(n, dtype=torch.int32, device=dev)
        self.tokens = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.host = [torch.zeros(n + batch, dtype=torch.int32).pin_memory() for _ in range(_RING)]
        self.host_views = [h.numpy() for h in self.host]   # the same pinned memory, for fast slice writes
        self.events = [None] * _RING
        self.turn = 0
        # host mirror of the block tables and which copies of it are current
        self.table_mirror = np.full((n_groups, batch, pages), -1, dtype=np.int32)
        self.table_rows = [[None] * batch for _ in range(n_groups)]
        self.table_version = 0                             # bumped whenever the mirror changes
        self.host_version = [-1] * _RING                   # version each staging buffer holds
        self.device_version = -1                           # version the device tables hold
        self.h2d_bytes = 0                                 # bytes copied host -> device so far
        self.staged_for = None                             # (sequences, lengths) whose next step is already on the device
        b = batch
        self.pos, self.total, self.slots = self.ints[0:b], self.ints[b:2 * b], self.ints[2 * b:3 * b]
        self.tables = {}
        at = 3 * b
        for g in cache.kv_groups:
            self.tables[g.index] = self.ints[at:at + b * pages].view(b, pages)
            at += b * pages
        arange = torch.arange(b + 1, dtype=torch.int32, device=dev)
        ones = torch.ones(b, dtype=torch.int32, device=dev)
        plan = AttentionPlan(n_seqs=b, max_new=1, max_total=self.capacity, all_single=True,
                             seq_start=self.pos, seq_new=ones, cu_new=arange, seq_total=self.total,
                             starts=[], news=[1] * b)
        self.ctx = StepContext(n_tokens=b, n_seqs=b, tokens=self.tokens, token_seq=arange[:b].contiguous(),
                               token_pos=self.pos, slots=self.slots, block_tables=self.tables,
                               want_rows=arange[:b].contiguous(), n_wanted=b, want_all=True,
                               attention_plan=plan, seq_start=self.pos, seq_new=ones, cu_new=arange)
        self.graph = None
        self.logits = None

    def stage(self, seqs, tokens, kv_groups, metadata=True):
        """Copy this step's positions, lengths, slots and block tables (``metadata``) and its tokens
        (when the host supplies them) to the device.  Fewer sequences than the graph has rows: the
        other rows are idle, each token 0 at position 0 of a sequence in the cache's idle slot and
        page, with a length of 0 after the step (`AttentionPlan.seq_total`): the decode attention
        gives it no work, whatever else runs on it stays in its own row."""
        i = self.turn
        self.turn = (self.turn + 1) % _RING
        if self.events[i] is not None:
            self.events[i].synchronize()                   # the copy that last used this buffer is done
        b, p = self.batch, self.pages
        if not metadata:
            host, view = self.host[i], self.host_views[i]
            n = 3 * b + self.table_mirror.size
            view[n:n + len(tokens)] = tokens
            view[n + len(tokens):n + b] = 0
            self.tokens.copy_(host[n:n + b], non_blocking=True)
            self.h2d_bytes += 4 * b
            ev = torch.cuda.Event()
            ev.record()
            self.events[i] = ev
            return
        idle = b - len(seqs)
        # Block tables change only when a sequence takes or gives back a page (or the batch changes):
        # keep a host mirror, rewrite the rows that changed, and send the tables only then.
        for gi, g in enumerate(kv_groups):
            for r in range(b):
                pages = seqs[r].pages[g.index] if r < len(seqs) else self.idle_pages
                if self.table_rows[gi][r] != pages:
                    self.table_mirror[gi, r, :len(pages)] = pages
                    self.table_mirror[gi, r, len(pages):] = -1
                    self.table_rows[gi][r] = list(pages)
                    self.table_version += 1
        host = self.host[i]
        view = self.host_views[i]
        small = 3 * b
        view[:b] = [s.length for s in seqs] + [0] * idle
        view[b:2 * b] = [s.length + 1 for s in seqs] + [0] * idle      # an idle row attends to nothing
        view[2 * b:small] = [s.slot for s in seqs] + [self.idle_slot] * idle
        n = small + self.table_mirror.size
        if self.device_version != self.table_version:
            if self.host_version[i] != self.table_version:
                view[small:n] = self.table_mirror.reshape(-1)
                self.host_version[i] = self.table_version
            self.ints.copy_(host[:n], non_blocking=True)
            self.device_version = self.table_version
            self.h2d_bytes += 4 * n
        else:
            self.ints[:small].copy_(host[:small], non_blocking=True)
            self.h2d_bytes += 4 * small
        if tokens is not None:
            view[n:n + len(tokens)] = tokens
            view[n + len(tokens):n + b] = 0
            self.tokens.copy_(host[n:n + b], non_blocking=True)
            self.h2d_bytes += 4 * b
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev

    def capture(self, model, cache):
        self.graph, self.logits = capture_forward(model, self.ctx, cache)


_capture_streams = {}          # device -> the side stream captures are made on


class CaptureFailed(RuntimeError):
    """The forward pass could not be captured as a CUDA graph (a part waited for the device or read
    device values on the host).  The cache is as it was before the step."""


def capture_forward(model, ctx, cache):
    """The forward pass of ``ctx`` as a CUDA graph: (graph, its logits buffer).  One eager run first:
    lazy allocations (counters, library workspaces) must not happen inside the capture.  It writes the
    keys and values the replay will write again; per-sequence state, which a second run would
    advance twice, is put back after it (`ModelCache.snapshot_state`).  The capture is begun and ended
    by hand on one side stream per device: the ready-made context manager empties the allocator's
    device and pinned-host caches at every entry, which cost 1 - 17 ms a capture here and once 1.3 s.
    Raises CaptureFailed, with the model marked not ``graph_safe``, if the pass cannot be captured."""
    device = model.runtime.device
    side = _capture_streams.get(device)
    if side is None:
        side = _capture_streams[device] = torch.cuda.Stream(device=device)
    current = torch.cuda.current_stream(device)
    side.wait_stream(current)
    graph = torch.cuda.CUDAGraph()
    failure = None
    with torch.cuda.stream(side):
        saved = cache.snapshot_state(ctx.slots)
        model.forward(ctx, cache)
        cache.restore_state(saved)
        torch.cuda.synchronize(device)
        if ctx.attention_plan is not None:
            ctx.attention_plan.scratch.clear()             # scratch must come from the graph's own pool
        graph.capture_begin()
        try:
            logits = model.forward(ctx, cache)
        except Exception as exc:                           # noqa: BLE001 - whatever the part raised, the capture must end
            failure = exc
        try:
            graph.capture_end()
        except RuntimeError as exc:
            failure = failure or exc
    current.wait_stream(side)
    if failure is not None:
        model.graph_safe = False
        torch.cuda.synchronize(device)
        if ctx.attention_plan is not None:
            ctx.attention_plan.scratch.clear()
        raise CaptureFailed(f"a step could not be captured as a CUDA graph ({type(failure).__name__}: {failure}); "
                            "the model runs its steps eagerly from now on.  A part whose forward waits for the "
                            "device or reads device values on the host declares graph_safe = False") from failure
    return graph, logits


LAUNCH_BOUND = 0.75            # host launch time / device time of an eager step from which a graph is worth its capture
LAUNCH_BOUND_PATIENCE = 8      # a device-bound batch size must come this many times as often before it is captured


def sightings_needed(capture_after, launch_share):
    """How many eager steps a batch size runs before it gets a graph.  A replayed graph saves the
    host's launches; where the device needs longer for the step than the host for launching it
    (``launch_share`` well below 1: large layers), the replay is no faster than the eager step, and
    a capture pays only for a batch size that stays for very long."""
    if launch_share is None or launch_share >= LAUNCH_BOUND:
        return capture_after
    return capture_after * LAUNCH_BOUND_PATIENCE


def graph_rows(batch):
    """Rows of the graph that serves ``batch`` sequences when one graph serves several batch sizes:
    the next power of two up to 16, the next multiple of 16 above.  The idle rows cost little: a
    decode step's time is the weights' and the live sequences' cache, read once whatever the rows,
    and the weight-streaming products work in steps of 16 rows anyway."""
    batch = int(batch)
    if batch <= 16:
        return 1 << max(0, batch - 1).bit_length()
    return (batch + 15) // 16 * 16


class DecodeGraphs:
    """Captured decode steps of one model and cache, by number of rows."""

    def __init__(self, model, cache):
        self.model = model
        self.cache = cache
        self.captured = {}
        self.captures = 0
        self.ahead_hits = 0                                # steps that found their positions and tables already sent
        self.eager_steps = {}                              # graph rows -> steps run eagerly while waiting to be worth a capture
        self.launch_share = None                           # of the last eager step: host time to launch it / device time to run it
        self._probe = None                                 # (start event, end event, host ms) of an eager step not yet read

    def takes(self, entries):
        return all(len(e.tokens) == 1 and (e.want is None or list(e.want) == [0]) for e in entries)

    def run(self, entries, device_tokens=False, capture_after=0, device_ids=None):
        """One decode step for ``entries`` (one token each).  Returns float32 logits [B, vocab] in a
        buffer that the next replay of the same batch size overwrites.  With ``device_tokens`` the
        tokens already in the graph's token buffer are used (``token_buffer(B)``), and the entries'
        tokens are ignored.  ``device_ids``: an int32 device tensor [B] with the tokens, copied into
        the graph's token buffer on the stream (the entries' tokens are ignored); with
        ``capture_after`` the call then returns None, having done nothing, when the width has no
        graph yet (an eager step needs its tokens on the host).

        ``capture_after`` (the generation loop's way): the step runs in a graph of `graph_rows(B)`
        rows whose other rows are idle (`_Captured.stage`), so that a batch that loses its requests
        one by one needs a graph per sixteen sizes and not per size; a width
        without a graph runs eagerly that many times before it is captured, and
        `LAUNCH_BOUND_PATIENCE` times as often while the eager steps are bound by the device and not
        by their launches (`sightings_needed`).  A capture costs two forward passes and 10 - 30 ms.
        64 requests of the 8B shape that ended five steps apart: 2.24 s eagerly; with a graph per
        batch size 3.64 s in the call that captured them and 1.56 s in the calls after it; with
        shared widths 1.96 s in the first call, captures included, and 1.54 s after it."""
        model, cache = self.model, self.cache
        seqs = [e.sequence for e in entries]
        b = rows = len(seqs)
        if capture_after and not device_tokens and b not in self.captured:
            rows = graph_rows(b)
            if rows not in self.captured:
                if device_ids is not None:
                    return None
                n = self.eager_steps.get(rows, 0)
                self._read_probe()
                if n < sightings_needed(capture_after, self.launch_share):
                    self.eager_steps[rows] = n + 1
                    return self._eager_step(entries)
        on_device = device_tokens or device_ids is not None
        slots = set()
        for i, (e, s) in enumerate(zip(entries, seqs)):
            if not getattr(s, "open", False):
                raise StepError(f"entry {i}: its sequence is closed")
            if s.slot in slots:
                raise StepError(f"entry {i}: slot {s.slot} occurs twice in one step")
            slots.add(s.slot)
            if s.length + 1 > model.spec.max_positions:
                raise StepError(f"entry {i}: position {s.length} is beyond the model's max positions "
                                f"{model.spec.max_positions}")
            if not on_device and not 0 <= int(e.tokens[0]) < model.spec.vocab_size:
                raise StepError(f"entry {i}: token id {e.tokens[0]} is outside the vocabulary")
        tokens = None if on_device else [int(e.tokens[0]) for e in entries]
        cap = self.captured.get(rows)
        if cap is not None and self._staged(cap, seqs, cache.kv_groups):
            # the step before this one already reserved the pages and sent everything but the tokens
            if tokens is not None:
                cap.stage(seqs, tokens, cache.kv_groups, metadata=False)
            self.ahead_hits += 1
            fresh = False
        else:
            cache.reserve([(s, s.length + 1) for s in seqs])
            pages = max(max((len(s.pages[g.index]) for g in cache.kv_groups), default=1) for s in seqs)
            fresh = cap is None or cap.pages < pages
            if fresh:
                room = min((model.spec.max_positions + PAGE - 1) // PAGE, max(pages + 16, (pages * 5) // 4))
                cap = _Captured(model, cache, rows, max(room, pages), len(cache.kv_groups))
                self.captured[rows] = cap
            cap.stage(seqs, tokens, cache.kv_groups)
        cap.staged_for = None
        if device_ids is not None:
            if device_ids.dtype != torch.int32 or device_ids.numel() != b:
                raise StepError(f"device_ids must be {b} int32 values")
            cap.tokens[:b].copy_(device_ids.reshape(-1), non_blocking=True)
        if fresh:
            try:
                cap.capture(model, cache)
            except CaptureFailed as exc:
                del self.captured[rows]
                if device_tokens:
                    raise
                warnings.warn(str(exc), RuntimeWarning, stacklevel=2)
                return None if device_ids is not None else self._eager_step(entries)
            self.captures += 1
        cap.graph.replay()
        for s in seqs:
            cache.commit(s, s.length + 1)
        self._stage_ahead(cap, seqs)
        return cap.logits if rows == b else cap.logits[:b]

    def _eager_step(self, entries):
        """The step without a graph, timed twice: the host's time to launch it and the device's time
        to run it (read at the next call, after the caller has waited for this step's result)."""
        from .step import run_step
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        start.record()
        logits = run_step(self.model, self.cache, entries)
        end.record()
        self._probe = (start, end, (time.perf_counter() - t0) * 1e3)
        return logits

    def _read_probe(self):
        if self._probe is not None and self._probe[1].query():
            start, end, host_ms = self._probe
            self._probe = None
            device_ms = start.elapsed_time(end)
            if device_ms > 0:
                self.launch_share = host_ms / device_ms

    @staticmethod
    def _staged(cap, seqs, kv_groups):
        """Is the device already set up for exactly these sequences at their present lengths, on the
        pages they hold now?  (A sequence that was truncated and has grown back to the staged length
        may hold other pages than the tables sent ahead name.)"""
        ahead = cap.staged_for
        if ahead is None or len(ahead[0]) != len(seqs):
            return False
        if not all(a is s and n == s.length for a, n, s in zip(ahead[0], ahead[1], seqs)):
            return False
        return all(cap.table_rows[gi][r] == s.pages[g.index]
                   for gi, g in enumerate(kv_groups) for r, s in enumerate(seqs))

    def _stage_ahead(self, cap, seqs):
        """While the device works on this step, send the next step's positions, lengths, slots and
        tables for the same sequences behind the running graph (same stream: they land after it has
        read the current ones), so that the next call only adds its tokens.  Only when no sequence
        needs a new page for its next token: nothing is reserved on a guess.  If the next call brings
        other sequences, or these at other lengths, it stages everything afresh."""
        model, cache = self.model, self.cache
        for s in seqs:
            if s.length + 1 > model.spec.max_positions or any(cache.pages_needed(s, s.length + 1).values()):
                return
        cap.stage(seqs, None, cache.kv_groups)
        cap.staged_for = (list(seqs), [s.length for s in seqs])

    def token_buffer(self, batch):
        """The device token buffer of the graph for ``batch`` sequences (after its first run)."""
        return self.captured[batch].tokens


class _CapturedStep:
    def __init__(self, buffer, ctx, graph, logits):
        self.buffer, self.ctx, self.graph, self.logits = buffer, ctx, graph, logits


class StepGraphs:
    """Captured steps of any shape (prompts, chunks), by shape.

    A prompt step is some hundred launches, and for a short prompt the host needs longer to launch
    them than the device to run them (128 tokens of the 8B sizes: 5.5 ms of launches, 3.3 ms of
    work); replayed from a graph the launches cost nothing and the gaps between dependent kernels go
    (2,048 tokens: 25.4 -> 23.6 ms).  A graph serves only steps of its own shape (tokens per sequence,
    number of wanted rows, table widths: the launch grids depend on them; where a sequence starts is
    data).  So that shapes repeat, block tables are as wide as sixteen pages need or a multiple of
    that (`table_widths`), and a sequence's tokens are filled up to a few lengths (`bucket_tokens`: powers of two
    up to 64, multiples of 64 up to 1,024) with tokens that are forgotten after the step
    (`_filled_up`); longer prompts run at their own length (fixed-size chunks, batches of equal
    prompts, benchmarks).  A shape is captured when it is seen for the second time; at most
    ``capacity`` graphs and ``row_budget`` token rows in all are kept (a graph holds the activations of
    its rows), the least recently used goes first.
    The same kernels run on the same data as in an eager step."""

    def __init__(self, model, cache, capacity=16, row_budget=1 << 15):
        self.model, self.cache, self.capacity, self.row_budget = model, cache, capacity, row_budget
        self.seen = {}
        self.captured = {}                                  # shape key -> _CapturedStep, in order of last use
        self.captures = 0
        self.replays = 0
        # Filling a sequence's tokens up and forgetting the rest afterwards needs a cache that can forget:
        # keys and values only (state cannot go back), no window (its pages may be gone by then).
        self.pads = all(g.kind == "kv" and not g.window for g in cache.groups)

    def _filled_up(self, entries):
        """The entries at the lengths a captured step runs them (`bucket_tokens`): token 0 after each
        one's own tokens.  Causal attention keeps those from every earlier row, and they are
        forgotten after the step (`ModelCache.truncate`), so the wanted logits and the cache are those
        of the step as it was asked for.  An entry stays as it is where the model's positions end."""
        from .step import StepEntry, bucket_tokens
        if not self.pads:
            return entries
        out = []
        for e in entries:
            n = len(e.tokens)
            room = bucket_tokens(n)
            if room == n or e.sequence.length + room > self.model.spec.max_positions:
                out.append(e)
                continue
            want = [n - 1] if e.want is None else list(e.want)
            out.append(StepEntry(e.sequence, [int(t) for t in e.tokens] + [0] * (room - n), want))
        return out

    def run(self, entries):
        """Logits float32 [wanted, vocab]; a replayed step returns a buffer that the next replay of the
        same shape overwrites."""
        from ..errors import CacheFullError
        from .step import plan_step, run_step, shape_key
        model, cache = self.model, self.cache
        filled = self._filled_up(entries)
        key = shape_key(filled, cache)
        cap = self.captured.get(key)
        if cap is None:
            self.seen[key] = self.seen.get(key, 0) + 1
            if self.seen[key] < 2 or len(self.seen) > 4096:
                if len(self.seen) > 4096:
                    self.seen.clear()
                return run_step(model, cache, entries)
            return self._capture(key, entries, filled)
        try:
            _, new_lengths = plan_step(filled, cache, model.spec.vocab_size, model.spec.max_positions,
                                       model.runtime.device, into=cap.buffer, widths=key[-1])
        except CacheFullError:
            return run_step(model, cache, entries)          # no room for the tokens that fill up: as asked for, eagerly
        except StepError as exc:
            if "does not fit" not in str(exc):
                raise
            del self.captured[key]                          # the sequences hold other page counts than the key foresaw
            return run_step(model, cache, entries)
        self.captured[key] = self.captured.pop(key)         # most recently used last
        cap.graph.replay()
        self.replays += 1
        self._commit(entries, filled, new_lengths)
        return cap.logits

    def _commit(self, entries, filled, new_lengths):
        """Record the step and forget the tokens that only filled it up."""
        for e, f, length in zip(entries, filled, new_lengths):
            self.cache.commit(e.sequence, length)
            extra = len(f.tokens) - len(e.tokens)
            if extra:
                self.cache.truncate(e.sequence, length - extra)

    def _capture(self, key, entries, filled):
        from ..errors import CacheFullError
        from .step import plan_step, run_step
        model, cache = self.model, self.cache
        try:
            ctx, new_lengths = plan_step(filled, cache, model.spec.vocab_size, model.spec.max_positions, model.runtime.device,
                                         widths=key[-1])
        except CacheFullError:
            return run_step(model, cache, entries)
        # the description moves into a buffer that stays: the graph's kernels read it at every replay
        buffer = torch.empty_like(ctx.packed)
        ctx, new_lengths = plan_step(filled, cache, model.spec.vocab_size, model.spec.max_positions,
                                     model.runtime.device, into=buffer, widths=key[-1])
        try:
            graph, logits = capture_forward(model, ctx, cache)
        except CaptureFailed as exc:
            warnings.warn(str(exc), RuntimeWarning, stacklevel=2)
            return run_step(model, cache, entries)
        graph.replay()                                      # the capture itself computes nothing
        self._commit(entries, filled, new_lengths)
        # room for the new graph: at most `capacity` graphs and `row_budget` token rows in all (a graph
        # holds the activations of its rows), the least recently used go first
        while self.captured and (len(self.captured) >= self.capacity or
                                 sum(c.ctx.n_tokens for c in self.captured.values()) + ctx.n_tokens > self.row_budget):
            self.captured.pop(next(iter(self.captured)))
        self.captured[key] = _CapturedStep(buffer, ctx, graph, logits)
        self.captures += 1
        return logits
