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
    seq_total: torch.Tensor       # int32 [B] length after the step
    starts: list = field(default_factory=list)
    news: list = field(default_factory=list)
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


def plan_step(entries, cache, vocab_size, max_positions, device):
    """Validate the entries, reserve cache room, and build the device-side description with one
    host-to-device copy.  Returns (StepContext, new lengths)."""
    if not entries:
        raise StepError("a step needs at least one sequence")
    seen = set()
    tokens, token_seq, token_pos, want_rows = [], [], [], []
    starts, news, slots = [], [], []
    offset = 0
    for b, e in enumerate(entries):
        seq = e.sequence
        if not getattr(seq, "open", False):
            raise StepError(f"entry {b}: its sequence is closed")
        if seq.slot in seen:
            raise StepError(f"entry {b}: slot {seq.slot} occurs twice in one step")
        seen.add(seq.slot)
        n = len(e.tokens)
        if n < 1:
            raise StepError(f"entry {b}: a sequence must bring at least one token")
        start = seq.length
        if start + n > max_positions:
            raise StepError(f"entry {b}: position {start + n - 1} is beyond the model's "
                            f"max positions {max_positions}")
        for t in e.tokens:
            if not 0 <= int(t) < vocab_size:
                raise StepError(f"entry {b}: token id {t} is outside the vocabulary [0, {vocab_size})")
        want = [n - 1] if e.want is None else list(e.want)
        for w in want:
            if not 0 <= int(w) < n:
                raise StepError(f"entry {b}: wanted offset {w} is outside its {n} tokens")
        tokens.extend(int(t) for t in e.tokens)
        token_seq.extend([b] * n)
        token_pos.extend(range(start, start + n))
        want_rows.extend(offset + int(w) for w in want)
        starts.append(start)
        news.append(n)
        slots.append(seq.slot)
        offset += n
    cache.reserve([(e.sequence, s + n) for e, s, n in zip(entries, starts, news)])

    T, B, R = offset, len(entries), len(want_rows)
    seqs = [e.sequence for e in entries]
    tables = {}
    for g in cache.kv_groups:
        rows, width = cache.block_table_rows(g.index, seqs)
        tables[g.index] = (rows, width)
    cu = [0]
    for n in news:
        cu.append(cu[-1] + n)
    # one packed int32 buffer, one copy
    totals = [s + n for s, n in zip(starts, news)]
    parts = [tokens, token_seq, token_pos, slots, starts, news, cu, want_rows, totals]
    for rows, width in tables.values():
        parts.append([p for row in rows for p in row])
    flat = [v for part in parts for v in part]
    host = torch.tensor(flat, dtype=torch.int32)
    if device.type == "cuda":
        host = host.pin_memory()
    dev = host.to(device, non_blocking=True)
    views = []
    at = 0
    for part in parts:
        views.append(dev[at:at + len(part)])
        at += len(part)
    d_tokens, d_seq, d_pos, d_slots, d_starts, d_news, d_cu, d_want, d_totals = views[:9]
    block_tables = {}
    for (gi, (rows, width)), view in zip(tables.items(), views[9:]):
        block_tables[gi] = view.view(B, width)
    plan = AttentionPlan(n_seqs=B, max_new=max(news), max_total=max(totals),
                         all_single=all(n == 1 for n in news), seq_start=d_starts, seq_new=d_news,
                         cu_new=d_cu, seq_total=d_totals, starts=starts, news=news)
    ctx = StepContext(n_tokens=T, n_seqs=B, tokens=d_tokens, token_seq=d_seq, token_pos=d_pos,
                      slots=d_slots, block_tables=block_tables, want_rows=d_want, n_wanted=R,
                      want_all=(R == T and want_rows == list(range(T))), attention_plan=plan,
                      seq_start=d_starts, seq_new=d_news, cu_new=d_cu)
    return ctx, totals


def run_step(model, cache, entries):
    """Logits float32 [wanted, vocab], in the order of the entries and of each entry's ``want``.
    On return every sequence's cached length has grown by the tokens it brought."""
    ctx, new_lengths = plan_step(entries, cache, model.spec.vocab_size, model.spec.max_positions,
                                 model.runtime.device)
    logits = model.forward(ctx, cache)
    for e, length in zip(entries, new_lengths):
        cache.commit(e.sequence, length)
    return logits
