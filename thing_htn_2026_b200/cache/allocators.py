"""Host-side bookkeeping of cache slots and pages.  No tensors, no device.

A *slot* stands for one live sequence.  A *page* holds ``page_size`` consecutive
positions of one sequence, for every cache entry of a group.  Both allocators hand out
the lowest free id first and refuse, with an exception, to free what is not held or to
hand out more than exists, so that a slot or page is never lost, held twice or freed
twice.

The reference keeps one cache row per batch row and rebuilds the cache when the batch
size changes (engine/engine.py:836-846); validity is by length only, stale contents are
never cleared (engine/kernels/torch_ref.py:211-215).  The same holds here: a reused slot
or page is not cleared.
"""

from __future__ import annotations

import heapq
from typing import Iterable, List


class CacheFull(RuntimeError):
    """Not enough free slots or pages for the request."""


class CacheStateError(RuntimeError):
    """An id was freed that is not held, or held twice: a bug in the caller."""


class IdAllocator:
    """Hands out integer ids from ``[0, capacity)``; lowest free id first."""

    def __init__(self, capacity: int, what: str):
        if capacity <= 0:
            raise ValueError(f"{what} allocator needs a positive capacity, got {capacity}")
        self.capacity = capacity
        self.what = what
        self._free: List[int] = list(range(capacity))
        heapq.heapify(self._free)
        self._held = set()

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return len(self._held)

    def held(self) -> frozenset:
        return frozenset(self._held)

    def take(self, count: int = 1) -> List[int]:
        if count < 0:
            raise ValueError(f"cannot take {count} {self.what}s")
        if count > len(self._free):
            raise CacheFull(f"need {count} {self.what}s, only {len(self._free)} of {self.capacity} are free")
        ids = [heapq.heappop(self._free) for _ in range(count)]
        self._held.update(ids)
        return ids

    def give_back(self, ids: Iterable[int]) -> None:
        ids = list(ids)
        if len(set(ids)) != len(ids):
            raise CacheStateError(f"{self.what} freed twice in one call: {sorted(ids)}")
        for i in ids:
            if i not in self._held:
                raise CacheStateError(f"{self.what} {i} is not held (freed twice, or never taken)")
        for i in ids:
            self._held.discard(i)
            heapq.heappush(self._free, i)

    def check(self) -> None:
        """Every id is either free or held, exactly once."""
        free = sorted(self._free)
        if len(set(free)) != len(free):
            raise CacheStateError(f"a {self.what} is on the free list twice")
        if set(free) & self._held:
            raise CacheStateError(f"a {self.what} is both free and held")
        if len(free) + len(self._held) != self.capacity:
            raise CacheStateError(
                f"{self.capacity - len(free) - len(self._held)} {self.what}s lost "
                f"({len(free)} free, {len(self._held)} held of {self.capacity})")
