"""Host-side bookkeeping of slots and pages.  Pure Python, no device work.

A slot is a sequence's row in the page tables and in every fixed-size state; a page is
`PAGE_TOKENS` cache entries of one group.  Both allocators refuse to hand out what is held
and to take back what is free, so that a slot or page can be neither lost, held twice nor
freed twice without an exception.
"""
from __future__ import annotations

import heapq


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    """No free slot, or not enough free pages."""


class IndexAllocator:
    """Hands out the lowest free index of 0..n-1."""

    def __init__(self, n, what="index"):
        self.n, self.what = n, what
        self._free = list(range(n))
        heapq.heapify(self._free)
        self._held = set()

    @property
    def free_count(self):
        return len(self._free)

    @property
    def held(self):
        return frozenset(self._held)

    def take(self, count=1):
        if count > len(self._free):
            raise CacheFull(f"{count} {self.what}(s) wanted, {len(self._free)} of {self.n} free")
        out = [heapq.heappop(self._free) for _ in range(count)]
        self._held.update(out)
        return out

    def give_back(self, indices):
        indices = list(indices)
        bad = [i for i in indices if i not in self._held]
        if bad or len(set(indices)) != len(indices):
            raise CacheError(f"{self.what}(s) {bad or indices} given back but not held")
        for i in indices:
            self._held.remove(i)
            heapq.heappush(self._free, i)
