"""The step function: run the tokens a batch of sequences brings, from the cache, and return
the logits at the wanted places.

The reference's ``IModel.Forward(tokenIds, positions, deviceId, kvCache)`` takes one sequence per
call: the whole prompt first, then one token per call
(src/DotLLM.Core/Models/IModel.cs:24-34, src/DotLLM.Engine/TextGenerator.cs:188,355).  Here one
call takes many sequences, each bringing its next tokens (a whole prompt, a chunk, or one token),
of unequal lengths, packed without padding.  Each sequence continues from its own cached length.
Only the given tokens are computed.  Everything is validated on the host before anything is
launched (token ids, positions, room in the cache; cf. TransformerModel.cs:137-143, 737-739 and
src/DotLLM.Engine/KvCache/SimpleKvCache.cs:78-80).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from ..errors import StepError


@dataclass
class StepEntry:
    """One sequence's share of a step: its next tokens and the offsets among them whose logits
    are wanted (``want`` None = the last token only; [] = none)."""
    sequence: object
    tokens: list
    want: Optional[list] = None


@dataclass
class AttentionPlan:
    """Layout of the step that the tensor-core attention kernels use (host numbers and device
    tensors shared by all layers of the step)."""
    n_seqs: int
    max_new: int                  # most new tokens any sequence brings
    max_total: int                # longest sequence after the step
    all_single: bool              # every sequence brings exactly one token (a decode step)
    seq_start: torch.Tensor       # int32 [B] cached length before the step
    seq_new: torch.Tensor         # int32 [B] tokens brought
    cu_new: torch.Tensor          # int32 [B+1] offsets of each sequence's tokens in the packed step
    seq_total: torch.Tensor       # int32 [B] length after the step; 0: an idle row (a captured step wider than
                                  # its batch), which attends to nothing and whose output nobody reads
    starts: list = field(default_factory=list)    # host copies of seq_start and seq_new, for scheduling only: a step replayed
    news: list = field(default_factory=list)      # from a graph carries the starts of the step it was captured from
    scratch: dict = field(default_factory=dict)


@dataclass
class StepContext:
    """Everything a part may need to know about the step, on the device."""
    n_tokens: int
    n_seqs: int
    tokens: torch.Tensor          # int32 [T]
    token_seq: torch.Tensor       # int32 [T] index of the token's sequence within the step
    token_pos: torch.Tensor       # int32 [T] absolute position of the token in its sequence
    slots: torch.Tensor           # int32 [B] cache slot of each sequence
    block_tables: dict            # kv group index -> int32 [B, P]
    want_rows: torch.Tensor       # int32 [R] packed row index of every wanted logit
    n_wanted: int
    want_all: bool
    attention_plan: Optional[AttentionPlan]
    seq_start: torch.Tensor       # int32 [B]
    seq_new: torch.Tensor         # int32 [B]
    cu_new: torch.Tensor          # int32 [B+1]
    packed: Optional[torch.Tensor] = None     # the one int32 device buffer all of the above are views of


PROMPT_PAD_LIMIT = 1024         # prompts (or chunks) of more tokens than this run at their own length in a captured step


def bucket_tokens(n):
    """The length at which a captured step runs ``n`` tokens of a sequence: the next power of two up to
    64, the next multiple of 64 up to `PROMPT_PAD_LIMIT`, ``n`` itself beyond (and for one token: a
    decode step).  The tokens that fill it up are run and then forgotten (`StepGraphs`)."""
    if n <= 1 or n > PROMPT_PAD_LIMIT:
        return n
    if n <= 64:
        return 1 << (n - 1).bit_length()
    return (n + 63) // 64 * 64


TABLE_WIDTH_STEP = 16           # a captured step's block tables are a multiple of this many pages wide


def shape_key(entries, cache):
    """What two steps must share for one captured graph to serve both: how many tokens each sequence
    brings, how many rows of each are wanted (and whether that is every row of the step), and how
    wide the block tables are (`table_widths`).  Launch shapes depend on these; the tokens, where a
    sequence starts, slots, page ids and which rows are wanted are data and do not enter."""
    news = tuple(len(e.tokens) for e in entries)
    wants = tuple(1 if e.want is None else len(e.want) for e in entries)
    every_row = all(e.want is not None and [int(w) for w in e.want] == list(range(len(e.tokens))) for e in entries)
    return news, wants, every_row, table_widths(entries, cache)


def table_widths(entries, cache):
    """Columns of a captured step's block table in every kv group: the pages of the longest sequence
    after the step, rounded up to `TABLE_WIDTH_STEP` (unused columns hold -1), so that a step's shape
    does not change with every page a sequence grows by."""
    pages = max(1, max((e.sequence.length + len(e.tokens) + 63) // 64 for e in entries))
    wide = (pages + TABLE_WIDTH_STEP - 1) // TABLE_WIDTH_STEP * TABLE_WIDTH_STEP
    return tuple(wide for _ in cache.kv_groups)


def plan_step(entries, cache, vocab_size, max_positions, device, into=None, widths=None):
    """Validate the entries, reserve cache room, and build the device-side description with one
    host-to-device copy.  Returns (StepContext, new lengths).  Per-token work is done on arrays, not
    in Python loops: a step may bring tens of thousands of prompt tokens.  ``into``: an int32 device
    buffer of exactly the description's size that receives it instead of a fresh one.  ``widths``:
    columns of the block table of every kv group, in the groups' order (at least the pages of the
    longest sequence; default: exactly those)."""
    if not entries:
        raise StepError("a step needs at least one sequence")
    B = len(entries)
    seen = set()
    starts = np.empty(B, dtype=np.int64)
    news = np.empty(B, dtype=np.int64)
    slots = np.empty(B, dtype=np.int64)
    token_arrays, want_arrays = [], []
    for b, e in enumerate(entries):
        seq = e.sequence
        if not getattr(seq, "open", False):
            raise StepError(f"entry {b}: its sequence is closed")
        if seq.slot in seen:
            raise StepError(f"entry {b}: slot {seq.slot} occurs twice in one step")
        seen.add(seq.slot)
        try:
            toks = np.asarray(e.tokens, dtype=np.int64).reshape(-1)
        except (TypeError, ValueError, OverflowError):
            raise StepError(f"entry {b}: its tokens are not integers") from None
        n = toks.size
        if n < 1:
            raise StepError(f"entry {b}: a sequence must bring at least one token")
        start = seq.length
        if start + n > max_positions:
            raise StepError(f"entry {b}: position {start + n - 1} is beyond the model's "
                            f"max positions {max_positions}")
        if toks.min() < 0 or toks.max() >= vocab_size:
            bad = toks[(toks < 0) | (toks >= vocab_size)][0]
            raise StepError(f"entry {b}: token id {int(bad)} is outside the vocabulary [0, {vocab_size})")
        want = np.asarray([n - 1] if e.want is None else e.want, dtype=np.int64).reshape(-1)
        if want.size and (want.min() < 0 or want.max() >= n):
            bad = want[(want < 0) | (want >= n)][0]
            raise StepError(f"entry {b}: wanted offset {int(bad)} is outside its {n} tokens")
        token_arrays.append(toks)
        want_arrays.append(want)
        starts[b], news[b], slots[b] = start, n, seq.slot
    totals = starts + news
    cache.reserve([(e.sequence, int(t)) for e, t in zip(entries, totals)])

    cu = np.zeros(B + 1, dtype=np.int64)
    np.cumsum(news, out=cu[1:])
    T = int(cu[-1])
    tokens = np.concatenate(token_arrays)
    token_seq = np.repeat(np.arange(B, dtype=np.int64), news)
    token_pos = np.arange(T, dtype=np.int64) - np.repeat(cu[:-1] - starts, news)
    want_rows = np.concatenate([w + cu[b] for b, w in enumerate(want_arrays)]) if want_arrays else np.zeros(0, np.int64)
    R = int(want_rows.size)
    seqs = [e.sequence for e in entries]
    tables = {}
    for gi, g in enumerate(cache.kv_groups):
        width = max(1, max(len(s.pages[g.index]) for s in seqs))
        if widths is not None:
            if widths[gi] < width:
                raise StepError(f"a block table of {widths[gi]} columns does not fit sequences of {width} pages")
            width = widths[gi]
        rows = np.full((B, width), -1, dtype=np.int64)
        for r, s in enumerate(seqs):
            pages = s.pages[g.index]
            rows[r, :len(pages)] = pages
        tables[g.index] = rows
    # one packed int32 buffer, one copy
    parts = [tokens, token_seq, token_pos, slots, starts, news, cu, want_rows, totals] + [t.reshape(-1) for t in tables.values()]
    sizes = [p.size for p in parts]
    host = torch.empty(sum(sizes), dtype=torch.int32, pin_memory=device.type == "cuda")
    view = host.numpy()
    at = 0
    for p, n in zip(parts, sizes):
        view[at:at + n] = p
        at += n
    if into is not None:
        # a captured step: the description goes into the buffer its graph reads (same layout: the
        # caller keys its graphs by `shape_key`)
        if into.numel() != host.numel():
            raise StepError("a captured step's buffer does not fit this step's description")
        into.copy_(host, non_blocking=True)
        dev = into
    else:
        dev = host.to(device, non_blocking=True)
    views = []
    at = 0
    for n in sizes:
        views.append(dev[at:at + n])
        at += n
    d_tokens, d_seq, d_pos, d_slots, d_starts, d_news, d_cu, d_want, d_totals = views[:9]
    block_tables = {gi: v.view(B, rows.shape[1]) for (gi, rows), v in zip(tables.items(), views[9:])}
    starts_l, news_l = starts.tolist(), news.tolist()
    plan = AttentionPlan(n_seqs=B, max_new=int(news.max()), max_total=int(totals.max()),
                         all_single=bool((news == 1).all()), seq_start=d_starts, seq_new=d_news,
                         cu_new=d_cu, seq_total=d_totals, starts=starts_l, news=news_l)
    ctx = StepContext(n_tokens=T, n_seqs=B, tokens=d_tokens, token_seq=d_seq, token_pos=d_pos,
                      slots=d_slots, block_tables=block_tables, want_rows=d_want, n_wanted=R,
                      want_all=bool(R == T and np.array_equal(want_rows, np.arange(T))), attention_plan=plan,
                      seq_start=d_starts, seq_new=d_news, cu_new=d_cu, packed=dev)
    return ctx, totals.tolist()


def run_step(model, cache, entries):
    """Logits float32 [wanted, vocab], in the order of the entries and of each entry's ``want``.
    On return every sequence's cached length has grown by the tokens it brought."""
    ctx, new_lengths = plan_step(entries, cache, model.spec.vocab_size, model.spec.max_positions,
                                 model.runtime.device)
    logits = model.forward(ctx, cache)
    for e, length in zip(entries, new_lengths):
        cache.commit(e.sequence, length)
    return logits
