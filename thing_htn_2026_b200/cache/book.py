"""Which sequence holds which slot and which pages: the host's view of the cache.

The cache is made of *groups*.  A group is a set of cache entries (one per layer that
writes a cache) with the same needs; it has storage and a page allocator of its own.
Two kinds of need exist for keys and values: all positions, or a window of the last W
positions.  A windowed group gives pages back as soon as every position in them has
fallen out of the window, so a long sequence holds about W / page_size pages there.

Each live sequence has a slot.  The slot indexes the per-sequence state of fixed size
(its length, and whatever else parts keep per sequence) and one row of every group's
block table: the physical page of each logical page (positions
``[i * page_size, (i + 1) * page_size)``), or -1.

This class only keeps the books and returns the block-table cells that changed; the
device mirror lives in :mod:`.sequence_cache`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

from .allocators import CacheFull, CacheStateError, IdAllocator

# (group, slot, logical page, physical page or -1)
TableUpdate = Tuple[int, int, int, int]


@dataclass(frozen=True)
class GroupBook:
    window: Optional[int]   # None: all positions are kept
    n_pages: int


class CacheBook:
    def __init__(self, groups: Sequence[GroupBook], page_size: int, max_slots: int, max_pages_per_seq: int):
        if page_size <= 0 or max_slots <= 0 or max_pages_per_seq <= 0:
            raise ValueError("page_size, max_slots and max_pages_per_seq must be positive")
        self.page_size = page_size
        self.max_slots = max_slots
        self.max_pages_per_seq = max_pages_per_seq
        self.groups = list(groups)
        self.slots = IdAllocator(max_slots, "slot")
        self.pages = [IdAllocator(g.n_pages, f"page of group {i}") for i, g in enumerate(self.groups)]
        self._length: Dict[int, int] = {}
        # per group: slot -> {logical page: physical page}
        self._held: List[Dict[int, Dict[int, int]]] = [dict() for _ in self.groups]

    # ------------------------------------------------------------------ slots

    def open(self) -> int:
        (slot,) = self.slots.take(1)
        self._length[slot] = 0
        for held in self._held:
            held[slot] = {}
        return slot

    def close(self, slot: int) -> List[TableUpdate]:
        if slot not in self._length:
            raise CacheStateError(f"slot {slot} is not open (closed twice, or never opened)")
        updates: List[TableUpdate] = []
        for g, held in enumerate(self._held):
            pages = held.pop(slot)
            self.pages[g].give_back(pages.values())
            updates.extend((g, slot, logical, -1) for logical in pages)
        del self._length[slot]
        self.slots.give_back([slot])
        return updates

    def is_open(self, slot: int) -> bool:
        return slot in self._length

    def length(self, slot: int) -> int:
        try:
            return self._length[slot]
        except KeyError:
            raise CacheStateError(f"slot {slot} is not open") from None

    def open_slots(self) -> List[int]:
        return sorted(self._length)

    # ------------------------------------------------------------------ pages

    def _first_needed_page(self, g: int, next_position: int) -> int:
        """Lowest logical page that a query at ``next_position`` or later can still read."""
        window = self.groups[g].window
        if window is None:
            return 0
        return max(0, next_position - window + 1) // self.page_size

    def pages_needed(self, slot: int, n_new: int) -> List[int]:
        """How many new pages each group needs to take ``n_new`` more tokens."""
        length = self.length(slot)
        if n_new <= 0:
            return [0] * len(self.groups)
        first, last = length // self.page_size, (length + n_new - 1) // self.page_size
        return [sum(1 for p in range(first, last + 1) if p not in self._held[g][slot])
                for g in range(len(self.groups))]

    def prepare(self, slots: Sequence[int], counts: Sequence[int]) -> List[TableUpdate]:
        """Map pages for the next ``counts[i]`` positions of ``slots[i]``.  All or nothing:
        on :class:`CacheFull` no page has been taken."""
        if len(set(slots)) != len(slots):
            raise CacheStateError(f"a slot appears twice in one step: {list(slots)}")
        need = [0] * len(self.groups)
        for slot, n in zip(slots, counts):
            if n < 0:
                raise ValueError(f"slot {slot}: cannot add {n} tokens")
            last_page = (self.length(slot) + n - 1) // self.page_size if n else -1
            if last_page >= self.max_pages_per_seq:
                raise CacheFull(
                    f"slot {slot}: {self.length(slot) + n} tokens exceed the longest sequence the cache was "
                    f"built for ({self.max_pages_per_seq * self.page_size})")
            for g, k in enumerate(self.pages_needed(slot, n)):
                need[g] += k
        for g, k in enumerate(need):
            if k > self.pages[g].n_free:
                raise CacheFull(
                    f"group {g}: step needs {k} more pages of {self.page_size} tokens, "
                    f"{self.pages[g].n_free} of {self.groups[g].n_pages} are free")
        updates: List[TableUpdate] = []
        for slot, n in zip(slots, counts):
            if n == 0:
                continue
            length = self._length[slot]
            first, last = length // self.page_size, (length + n - 1) // self.page_size
            for g in range(len(self.groups)):
                held = self._held[g][slot]
                missing = [p for p in range(first, last + 1) if p not in held]
                for logical, physical in zip(missing, self.pages[g].take(len(missing))):
                    held[logical] = physical
                    updates.append((g, slot, logical, physical))
        return updates

    def commit(self, slots: Sequence[int], counts: Sequence[int]) -> List[TableUpdate]:
        """The step's tokens are in the cache: lengths grow; windowed groups give back the
        pages that no later query can read."""
        updates: List[TableUpdate] = []
        for slot, n in zip(slots, counts):
            new_length = self.length(slot) + n
            if (new_length + self.page_size - 1) // self.page_size > self.max_pages_per_seq:
                raise CacheStateError(f"slot {slot}: commit beyond the prepared pages")
            self._length[slot] = new_length
            for g in range(len(self.groups)):
                keep_from = self._first_needed_page(g, new_length)
                if keep_from == 0:
                    continue
                held = self._held[g][slot]
                gone = [p for p in held if p < keep_from]
                if gone:
                    self.pages[g].give_back(held.pop(p) for p in gone)
                    updates.extend((g, slot, p, -1) for p in gone)
        return updates

    def pages_of(self, g: int, slot: int) -> Dict[int, int]:
        return dict(self._held[g][slot])

    def tokens_held(self) -> int:
        """Tokens of live sequences, each rounded up to whole pages."""
        return sum(-(-n // self.page_size) * self.page_size for n in self._length.values())

    # ------------------------------------------------------------------ invariants

    def check(self) -> None:
        self.slots.check()
        if set(self._length) != set(self.slots.held()):
            raise CacheStateError("open sequences and held slots differ")
        for g, alloc in enumerate(self.pages):
            alloc.check()
            seen = []
            for slot, pages in self._held[g].items():
                if slot not in self._length:
                    raise CacheStateError(f"group {g}: pages recorded for closed slot {slot}")
                seen.extend(pages.values())
            if len(set(seen)) != len(seen):
                raise CacheStateError(f"group {g}: a page is mapped twice")
            if set(seen) != set(alloc.held()):
                raise CacheStateError(f"group {g}: mapped pages and held pages differ")
