"""A pool of integer ids (cache slots, cache pages) that are handed out and given back.

Invariant: every id is either free or held, never both, never neither; freeing an id that is
not held, or twice, is an error and changes nothing.
"""
from __future__ import annotations

from ..errors import CacheError, CacheFullError


class IdPool:
    def __init__(self, count, what="id"):
        if count < 0:
            raise CacheError(f"a pool cannot hold {count} {what}s")
        self.count = int(count)
        self.what = what
        self._free = list(range(self.count - 1, -1, -1))     # pop() hands out 0 first
        self._held = set()

    @property
    def n_free(self):
        return len(self._free)

    @property
    def n_held(self):
        return len(self._held)

    def held(self):
        return frozenset(self._held)

    def free_ids(self):
        return list(self._free)

    def alloc(self):
        if not self._free:
            raise CacheFullError(f"no free {self.what} (all {self.count} are held)")
        i = self._free.pop()
        self._held.add(i)
        return i

    def alloc_many(self, n):
        """All or nothing: either ``n`` ids or CacheFullError with the pool unchanged."""
        if n > len(self._free):
            raise CacheFullError(f"need {n} {self.what}s, only {len(self._free)} of {self.count} are free")
        return [self.alloc() for _ in range(n)]

    def free(self, i):
        if i not in self._held:
            raise CacheError(f"{self.what} {i} is not held (freed twice, or never handed out)")
        self._held.remove(i)
        self._free.append(i)        # most recently freed is reused first

    def check(self):
        """Raise if the invariant is broken (used by tests)."""
        free = set(self._free)
        if len(free) != len(self._free) or free & self._held or free | self._held != set(range(self.count)):
            raise CacheError(f"{self.what} pool corrupted: free={sorted(free)} held={sorted(self._held)}")
