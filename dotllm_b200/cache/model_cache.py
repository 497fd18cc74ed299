"""The cache of a model: one slot per live sequence, storage per group of layers.

The reference keeps one ``SimpleKvCache`` per sequence, per layer a K and a V buffer of
``[maxLen, nkv*hd]`` written at ``positions[i]`` (src/DotLLM.Engine/KvCache/SimpleKvCache.cs:40-98).
Here one object serves a batch:

* a *slot* per live sequence (``Sequence``), handed out when the sequence opens and given back
  when it closes, with the sequence's own length;
* per *group* of layer executions with equal needs, storage of its own.  A "kv" group holds keys
  and values in pages of 64 tokens taken from the group's pool as the sequence grows (K page
  ``[kv_head][token][key width]``, V page ``[kv_head][value width][token]``, in the group's own
  storage type when its mixer asks for one); a group with a window gives pages
  back once every token in them is older than the window.  A "state" group holds a fixed-size
  tensor per slot, zeroed when a sequence opens;
* an execution that reads another execution's cache gets a view of that storage and never writes;
* one slot and one page per group beyond those the pools hand out (``idle_slot``, ``idle_page``): a
  step whose launch shapes are wider than its batch (a captured decode step that serves several
  batch sizes) points its idle rows there, as sequences of one token whose results nobody reads.
  No live sequence ever holds them, so what idle rows write reaches no result.

Pages are counted in tokens: ``max_tokens`` is the most tokens live sequences may hold at once,
each sequence's count rounded up to a whole page.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ..errors import CacheError, CacheFullError
from .pool import IdPool

PAGE = 64


@dataclass
class Sequence:
    """A live sequence: its slot, how many tokens it holds, and its pages in every kv group."""
    slot: int
    length: int = 0
    pages: dict = field(default_factory=dict)      # group index -> list of page ids (-1 = given back)
    open: bool = True


@dataclass
class LayerCacheView:
    """What a mixer sees of the cache during one step."""
    kind: str
    writes: bool
    k: Optional[torch.Tensor] = None               # [pages, nkv, 64, hd]
    v: Optional[torch.Tensor] = None               # [pages, nkv, hd, 64]
    block_table: Optional[torch.Tensor] = None     # int32 [B, P]: page of sequence b's tokens 64p..64p+63
    state: Optional[torch.Tensor] = None           # [slots, *state_shape]
    slots: Optional[torch.Tensor] = None           # int32 [B]: slot of each sequence of the step


class CacheGroup:
    def __init__(self, index, need, entries, runtime, n_pages, n_slots):
        self.index = index
        self.need = need
        self.kind = need.kind
        self.entries = list(entries)                # schedule entries that own storage here
        self.local = {e: i for i, e in enumerate(self.entries)}
        n = len(self.entries)
        if self.kind == "kv":
            self.window = need.window
            self.pages = IdPool(n_pages, "page")
            dtype = need.dtype or runtime.dtype
            # one page more than the pool hands out: the cache's idle page
            self.k = torch.zeros((n, n_pages + 1, need.n_kv_heads, PAGE, need.key_width()), dtype=dtype, device=runtime.device)
            self.v = torch.zeros((n, n_pages + 1, need.n_kv_heads, need.value_width(), PAGE), dtype=dtype, device=runtime.device)
            self.state = None
        elif self.kind == "state":
            self.window = None
            self.pages = None
            self.k = self.v = None
            self.state = torch.zeros((n, n_slots + 1, *need.state_shape), dtype=need.state_dtype,
                                     device=runtime.device)    # one slot more: the cache's idle slot
        else:
            raise CacheError(f"unknown cache kind {need.kind!r}")

    def bytes(self):
        if self.kind == "kv":
            return (self.k.numel() + self.v.numel()) * self.k.element_size()
        return self.state.numel() * self.state.element_size()

    def bytes_per_token(self):
        """Bytes of keys and values one cached token takes in this group."""
        if self.kind != "kv":
            return 0
        return len(self.entries) * self.need.n_kv_heads * (self.need.key_width() + self.need.value_width()) * self.k.element_size()


class ModelCache:
    """``needs[e]`` is the CacheNeed of schedule entry e (None: keeps nothing); ``cache_of[e]`` is
    None or the earlier entry whose storage entry e reads."""

    def __init__(self, needs, cache_of, runtime, max_tokens, max_sequences=None):
        if max_tokens <= 0:
            raise CacheError("max_tokens must be positive")
        self.runtime = runtime
        self.n_pages = (int(max_tokens) + PAGE - 1) // PAGE
        self.max_tokens = self.n_pages * PAGE
        # every live sequence holds at least one page, so more slots than pages are never used
        self.n_slots = int(max_sequences) if max_sequences else self.n_pages
        self.slots = IdPool(self.n_slots, "slot")
        self.idle_slot, self.idle_page = self.n_slots, self.n_pages      # never handed out
        self.groups = []
        self.entry_group = {}                       # schedule entry -> (group index, owner entry)
        by_key = {}
        for e, need in enumerate(needs):
            owner = cache_of[e] if cache_of[e] is not None else e
            if owner != e:
                continue
            if need is None:
                continue
            by_key.setdefault(need.group_key(runtime.dtype), (need, []))[1].append(e)
        for key, (need, entries) in by_key.items():
            self.groups.append(CacheGroup(len(self.groups), need, entries, runtime, self.n_pages, self.n_slots))
        for g in self.groups:
            for e in g.entries:
                self.entry_group[e] = (g.index, e)
        for e, need in enumerate(needs):
            owner = cache_of[e]
            if owner is not None:
                if owner not in self.entry_group:
                    raise CacheError(f"schedule entry {e} reads the cache of entry {owner}, which keeps none")
                self.entry_group[e] = (self.entry_group[owner][0], owner)
        self.kv_groups = [g for g in self.groups if g.kind == "kv"]
        self.live = {}                              # slot -> Sequence

    # ------------------------------------------------------------ sequences
    def open_sequence(self):
        slot = self.slots.alloc()
        seq = Sequence(slot=slot, pages={g.index: [] for g in self.kv_groups})
        for g in self.groups:
            if g.kind == "state":
                g.state[:, slot].zero_()
        self.live[slot] = seq
        return seq

    def close_sequence(self, seq):
        if not seq.open or self.live.get(seq.slot) is not seq:
            raise CacheError(f"sequence in slot {seq.slot} is not open (closed twice?)")
        for g in self.kv_groups:
            for page in seq.pages[g.index]:
                if page >= 0:
                    g.pages.free(page)
            seq.pages[g.index] = []
        self.slots.free(seq.slot)
        del self.live[seq.slot]
        seq.open = False
        seq.length = 0

    def pages_needed(self, seq, new_length):
        """Pages each kv group must still hand out so that ``seq`` can hold ``new_length`` tokens."""
        want = (new_length + PAGE - 1) // PAGE
        return {g.index: max(0, want - len(seq.pages[g.index])) for g in self.kv_groups}

    def reserve(self, seqs_and_lengths):
        """Make room for every (sequence, new length) of a step, or raise CacheFullError and
        change nothing."""
        demand = {g.index: 0 for g in self.kv_groups}
        for seq, new_length in seqs_and_lengths:
            if not seq.open:
                raise CacheError(f"sequence in slot {seq.slot} is closed")
            for gi, n in self.pages_needed(seq, new_length).items():
                demand[gi] += n
        for g in self.kv_groups:
            if demand[g.index] > g.pages.n_free:
                raise CacheFullError(
                    f"the step needs {demand[g.index]} more pages of {PAGE} tokens in cache group "
                    f"{g.index}, only {g.pages.n_free} of {g.pages.count} are free "
                    f"(cache sized for {self.max_tokens} tokens)")
        for seq, new_length in seqs_and_lengths:
            for gi, n in self.pages_needed(seq, new_length).items():
                seq.pages[gi].extend(self.groups[gi].pages.alloc_many(n))

    def commit(self, seq, new_length):
        """The step wrote tokens up to ``new_length``: record it and give back pages that a
        windowed group no longer needs."""
        if new_length < seq.length:
            raise CacheError("a sequence cannot shrink in a step")
        seq.length = new_length
        for g in self.kv_groups:
            if g.window:
                oldest_needed = new_length - g.window + 1       # first key the next query may see
                pages = seq.pages[g.index]
                for p in range(len(pages)):
                    if pages[p] >= 0 and PAGE * p + PAGE - 1 < oldest_needed:
                        g.pages.free(pages[p])
                        pages[p] = -1

    def truncate(self, seq, length):
        """Forget tokens beyond ``length`` (the reference's Rollback,
        src/DotLLM.Engine/KvCache/SimpleKvCache.cs:139-152).  Windowed groups cannot go back
        past pages they have given up."""
        if length < 0 or length > seq.length:
            raise CacheError(f"cannot truncate a sequence of {seq.length} tokens to {length}")
        keep = (length + PAGE - 1) // PAGE
        for g in self.kv_groups:
            pages = seq.pages[g.index]
            if g.window and any(p < 0 for p in pages[max(0, (length - g.window + 1)) // PAGE:keep]):
                raise CacheError("a windowed cache group has already given up pages this truncation needs")
            for page in pages[keep:]:
                if page >= 0:
                    g.pages.free(page)
            del pages[keep:]
        seq.length = length

    # ---------------------------------------------------------------- views
    def block_table_rows(self, group_index, seqs):
        """Host lists of page ids, one per sequence, padded with -1 to a common width."""
        width = max(1, max(len(s.pages[group_index]) for s in seqs))
        return [s.pages[group_index] + [-1] * (width - len(s.pages[group_index])) for s in seqs], width

    def view(self, entry, block_tables, slots):
        """The storage of schedule entry ``entry`` for this step.  ``block_tables[g]`` is the
        step's device block table of kv group g; ``slots`` the device slot ids of its sequences."""
        if entry not in self.entry_group:
            return None
        gi, owner = self.entry_group[entry]
        g = self.groups[gi]
        local = g.local[owner]
        writes = owner == entry
        if g.kind == "kv":
            return LayerCacheView("kv", writes, k=g.k[local], v=g.v[local], block_table=block_tables[gi])
        return LayerCacheView("state", writes, state=g.state[local], slots=slots)

    def snapshot_state(self, slots):
        """Copies of the fixed-size state of the given slots (an int32 device tensor), for a step that
        has to run twice (the trial run before a graph capture).  Keys and values need none: a second
        run writes the same values to the same places."""
        index = slots.long()
        return [(g, index, g.state[:, index].clone()) for g in self.groups if g.kind == "state"]

    @staticmethod
    def restore_state(saved):
        for g, index, values in saved:
            g.state[:, index] = values

    # ---------------------------------------------------------------- admin
    def bytes(self):
        return sum(g.bytes() for g in self.groups)

    def bytes_per_token(self):
        return sum(g.bytes_per_token() for g in self.groups)

    def free_tokens(self):
        """Tokens' worth of free pages in the tightest kv group."""
        return min((g.pages.n_free for g in self.kv_groups), default=self.n_pages) * PAGE

    def check(self):
        """Raise if a slot or page is lost, held twice, or held by no live sequence (tests)."""
        self.slots.check()
        if set(self.live) != set(self.slots.held()):
            raise CacheError(f"live sequences {sorted(self.live)} do not match held slots "
                             f"{sorted(self.slots.held())}")
        for g in self.kv_groups:
            g.pages.check()
            owned = [p for s in self.live.values() for p in s.pages[g.index] if p >= 0]
            if len(owned) != len(set(owned)):
                raise CacheError(f"group {g.index}: a page is held by two sequences")
            if set(owned) != set(g.pages.held()):
                raise CacheError(f"group {g.index}: held pages {sorted(g.pages.held())} do not match "
                                 f"the pages of live sequences {sorted(owned)}")

    def fill_free_pages(self, value):
        """Overwrite every page that no sequence holds (tests use NaN to show that stale data
        never reaches a result)."""
        for g in self.kv_groups:
            ids = g.pages.free_ids()
            if ids:
                index = torch.tensor(ids, dtype=torch.long, device=g.k.device)
                g.k[:, index] = value
                g.v[:, index] = value
