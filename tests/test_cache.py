"""The cache on the CPU: no slot or page lost, held twice or freed twice; groups; windows; state."""
import random

import pytest
import torch

from dotllm_b200.cache import IdPool, ModelCache, PAGE
from dotllm_b200.errors import CacheError, CacheFullError
from dotllm_b200.parts.base import CacheNeed, Runtime

CPU = Runtime(torch.float32, torch.device("cpu"))
KV = CacheNeed("kv", n_kv_heads=2, head_dim=16)


def test_id_pool_invariants():
    pool = IdPool(4, "slot")
    ids = [pool.alloc() for _ in range(4)]
    assert sorted(ids) == [0, 1, 2, 3] and pool.n_free == 0
    with pytest.raises(CacheFullError):
        pool.alloc()
    pool.free(2)
    with pytest.raises(CacheError, match="not held"):
        pool.free(2)                                     # freed twice
    with pytest.raises(CacheError):
        pool.free(7)                                     # never handed out
    assert pool.alloc() == 2                             # given back, used again
    pool.check()
    with pytest.raises(CacheFullError):
        IdPool(3).alloc_many(4)
    p = IdPool(3)
    with pytest.raises(CacheFullError):
        p.alloc_many(4)
    assert p.n_free == 3                                 # all or nothing


def test_random_open_grow_close_never_loses_anything():
    cache = ModelCache([KV, KV, KV], [None, None, None], CPU, max_tokens=64 * 12)
    rng = random.Random(0)
    live = []
    for _ in range(400):
        action = rng.random()
        if action < 0.35 and cache.slots.n_free:
            live.append(cache.open_sequence())
        elif action < 0.8 and live:
            s = rng.choice(live)
            new = s.length + rng.randint(1, 90)
            try:
                cache.reserve([(s, new)])
                cache.commit(s, new)
            except CacheFullError:
                pass
        elif live:
            s = live.pop(rng.randrange(len(live)))
            cache.close_sequence(s)
            with pytest.raises(CacheError):
                cache.close_sequence(s)                  # closed twice
        cache.check()
        held = sum(len(s.pages[0]) for s in live)
        assert held == cache.groups[0].pages.n_held
        assert all(len(s.pages[0]) == (s.length + PAGE - 1) // PAGE for s in live)
    for s in live:
        cache.close_sequence(s)
    cache.check()
    assert cache.slots.n_free == cache.n_slots and cache.groups[0].pages.n_free == cache.n_pages


def test_reserve_is_all_or_nothing_and_counts_in_pages():
    cache = ModelCache([KV], [None], CPU, max_tokens=64 * 3)
    a, b = cache.open_sequence(), cache.open_sequence()
    cache.reserve([(a, 65)])                             # two pages
    cache.commit(a, 65)
    with pytest.raises(CacheFullError, match="pages"):
        cache.reserve([(a, 129), (b, 1)])                # needs two more, one is free
    assert len(a.pages[0]) == 2 and len(b.pages[0]) == 0 and cache.groups[0].pages.n_free == 1
    cache.reserve([(b, 64)])
    assert cache.free_tokens() == 0
    cache.close_sequence(a)
    assert cache.free_tokens() == 128
    c = cache.open_sequence()
    assert c.slot == a.slot and c.length == 0           # the slot is used again, empty


def test_groups_follow_needs_and_shared_caches():
    full = CacheNeed("kv", n_kv_heads=2, head_dim=16)
    windowed = CacheNeed("kv", n_kv_heads=2, head_dim=16, window=100)
    other = CacheNeed("kv", n_kv_heads=1, head_dim=32)
    state = CacheNeed("state", state_shape=(3, 5), state_dtype=torch.float32)
    needs = [full, windowed, full, other, state, None, full]
    cache_of = [None, None, None, None, None, None, 0]   # the last execution reads entry 0's cache
    cache = ModelCache(needs, cache_of, CPU, max_tokens=64 * 8, max_sequences=4)
    kinds = sorted((g.kind, len(g.entries)) for g in cache.groups)
    assert kinds == [("kv", 1), ("kv", 1), ("kv", 2), ("state", 1)]
    s = cache.open_sequence()
    cache.reserve([(s, 10)])
    tables = {g.index: torch.tensor(cache.block_table_rows(g.index, [s])[0], dtype=torch.int32)
              for g in cache.kv_groups}
    slots = torch.tensor([s.slot], dtype=torch.int32)
    v0, v6, v5, v4 = (cache.view(e, tables, slots) for e in (0, 6, 5, 4))
    assert v0.writes and not v6.writes and v6.k.data_ptr() == v0.k.data_ptr()
    assert v5 is None
    assert v4.kind == "state" and v4.state.shape == (4 + 1, 3, 5)          # the four slots and the idle one
    assert cache.view(2, tables, slots).k.data_ptr() != v0.k.data_ptr()
    with pytest.raises(CacheError):
        ModelCache([None, full], [None, 0], CPU, max_tokens=64)     # reads a cache that does not exist


def test_windowed_group_gives_pages_back_and_state_is_zeroed():
    windowed = CacheNeed("kv", n_kv_heads=1, head_dim=16, window=70)
    full = CacheNeed("kv", n_kv_heads=1, head_dim=16)
    state = CacheNeed("state", state_shape=(4,))
    cache = ModelCache([windowed, full, state], [None, None, None], CPU, max_tokens=64 * 10)
    gw = next(g for g in cache.kv_groups if g.window)
    gf = next(g for g in cache.kv_groups if not g.window)
    s = cache.open_sequence()
    cache.groups[2].state[0, s.slot] = 7.0
    for length in (64, 128, 200, 300):
        cache.reserve([(s, length)])
        cache.commit(s, length)
        cache.check()
    # keys older than 300 - 70 + 1 = 231 are not needed: pages 0..2 (tokens < 192) are given back
    assert s.pages[gw.index][:3] == [-1, -1, -1] and all(p >= 0 for p in s.pages[gw.index][3:])
    assert gw.pages.n_held == 2 and gf.pages.n_held == 5
    slot = s.slot
    cache.close_sequence(s)
    again = cache.open_sequence()
    assert again.slot == slot and float(cache.groups[2].state[0, slot].abs().sum()) == 0.0
    cache.check()


def test_truncate():
    cache = ModelCache([KV], [None], CPU, max_tokens=64 * 4)
    s = cache.open_sequence()
    cache.reserve([(s, 200)])
    cache.commit(s, 200)
    cache.truncate(s, 65)
    assert s.length == 65 and len(s.pages[0]) == 2 and cache.groups[0].pages.n_free == 2
    with pytest.raises(CacheError):
        cache.truncate(s, 66)
    cache.check()


def test_idle_slot_and_page_lie_outside_the_pools_and_state_can_be_put_back():
    """The cache keeps one slot and one page per group that its pools never hand out (the idle rows of
    a step wider than its batch work there), and the fixed-size state of given slots can be copied
    and put back (a step that has to run twice must not advance it twice)."""
    kv = CacheNeed("kv", n_kv_heads=1, head_dim=16)
    state = CacheNeed("state", state_shape=(3,), state_dtype=torch.float32)
    cache = ModelCache([kv, state], [None, None], CPU, max_tokens=64 * 4, max_sequences=2)
    assert cache.idle_slot == 2 and cache.idle_page == 4
    seqs = [cache.open_sequence() for _ in range(2)]
    cache.reserve([(s, 128) for s in seqs])
    assert cache.idle_slot not in {s.slot for s in seqs}
    assert all(cache.idle_page not in s.pages[g.index] for s in seqs for g in cache.kv_groups)
    for g in cache.kv_groups:
        assert g.k.shape[1] == 4 + 1 and g.pages.n_free == 0       # every page of the pool is out, the idle one is not of it
    group = [g for g in cache.groups if g.kind == "state"][0]
    assert group.state.shape == (1, 2 + 1, 3)
    group.state[0, seqs[1].slot] = torch.tensor([1.0, 2.0, 3.0])
    slots = torch.tensor([seqs[1].slot, cache.idle_slot], dtype=torch.int32)
    saved = cache.snapshot_state(slots)
    group.state[0, seqs[1].slot] += 5.0
    group.state[0, cache.idle_slot] = 9.0
    group.state[0, seqs[0].slot] = 7.0                              # not among the saved slots: stays
    cache.restore_state(saved)
    assert group.state[0, seqs[1].slot].tolist() == [1.0, 2.0, 3.0]
    assert group.state[0, cache.idle_slot].tolist() == [0.0, 0.0, 0.0]
    assert group.state[0, seqs[0].slot].tolist() == [7.0, 7.0, 7.0]
    cache.check()
