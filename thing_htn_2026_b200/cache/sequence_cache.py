"""The cache on the device: paged keys and values per group of layers, per-sequence state
of fixed size, and the device copies of block tables and lengths.

Storage of a key/value group: ``[entries, pages, 2, n_kv, page_size, head_dim]`` (K then
V inside a page, head-major, so the ``page_size * head_dim`` values of one head of one
page are contiguous).  The reference's layout is ``[B, Nkv, CAP, D]`` per layer
(engine/engine.py:844-846); pages replace the fixed capacity so that sequences of very
different lengths share one pool.

Per-sequence state of fixed size lives in tensors ``[max_slots, ...]`` indexed by slot:
``seq_lens`` (tokens in the cache = next position; the reference's ``pos_buf``,
engine/engine.py:849) and any state a part or the generation loop registers.  Opening a
slot resets its row of every such tensor; pages are never cleared (validity is by
length, as in the reference, engine/kernels/torch_ref.py:211-215).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

from .. import ops
from .allocators import CacheFull
from .book import CacheBook, GroupBook, TableUpdate

PAGE_SIZE = 64


@dataclass(frozen=True)
class KVSpec:
    """A mixer's need for keys and values: ``window=None`` keeps all positions."""

    n_kv: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """A mixer's need for per-sequence state of fixed size (zeroed when a slot opens)."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


CacheNeed = Union[KVSpec, StateSpec, None]


class SequenceCache:
    def __init__(self, needs: Sequence[CacheNeed], *, max_tokens: int, dtype: torch.dtype, device,
                 max_slots: Optional[int] = None, max_seq_len: Optional[int] = None,
                 page_size: int = PAGE_SIZE):
        """``needs[e]`` is what cache entry ``e`` stores.  ``max_tokens`` is the most tokens
        that live sequences hold together, each sequence rounded up to whole pages."""
        self.device = torch.device(device)
        self.dtype = dtype
        self.page_size = page_size
        n_pages = max(1, -(-int(max_tokens) // page_size))
        self.max_slots = int(max_slots) if max_slots else min(n_pages, 1024)
        longest = n_pages if max_seq_len is None else min(n_pages, -(-int(max_seq_len) // page_size))
        self.max_pages_per_seq = max(1, longest)

        # group the entries by need
        self.kv_specs: List[KVSpec] = []
        self._entry_place: Dict[int, Tuple[str, int, int]] = {}   # entry -> (kind, group, index in group)
        state_specs: List[StateSpec] = []
        counts: Dict[Tuple[str, int], int] = {}
        for entry, need in enumerate(needs):
            if need is None:
                continue
            if isinstance(need, KVSpec):
                if need not in self.kv_specs:
                    self.kv_specs.append(need)
                key = ("kv", self.kv_specs.index(need))
            elif isinstance(need, StateSpec):
                if need not in state_specs:
                    state_specs.append(need)
                key = ("state", state_specs.index(need))
            else:
                raise TypeError(f"cache entry {entry}: unknown need {need!r}")
            self._entry_place[entry] = (key[0], key[1], counts.get(key, 0))
            counts[key] = counts.get(key, 0) + 1

        self.book = CacheBook([GroupBook(spec.window, n_pages) for spec in self.kv_specs], page_size,
                              self.max_slots, self.max_pages_per_seq)
        # Zeroed once: pages are never cleared afterwards, but what lies beyond a sequence's
        # length must stay finite (a masked key's weight is 0, and 0 * NaN would poison V).
        self.kv_storage = [
            torch.zeros((counts[("kv", g)], n_pages, 2, spec.n_kv, page_size, spec.head_dim), dtype=dtype,
                        device=self.device)
            for g, spec in enumerate(self.kv_specs)
        ]
        self.block_tables = [torch.full((self.max_slots, self.max_pages_per_seq), -1, dtype=torch.int32,
                                        device=self.device) for _ in self.kv_specs]
        self.state_storage = [
            torch.zeros((counts[("state", g)], self.max_slots, *spec.shape), dtype=spec.dtype, device=self.device)
            for g, spec in enumerate(state_specs)
        ]
        self.seq_lens = torch.zeros(self.max_slots, dtype=torch.int32, device=self.device)
        self._named_state: Dict[str, torch.Tensor] = {}
        self.n_pages = n_pages

    # ------------------------------------------------------------------ per-sequence state

    def sequence_state(self, name: str, shape: Tuple[int, ...] = (), dtype: torch.dtype = torch.int32) -> torch.Tensor:
        """A named tensor ``[max_slots, *shape]``; a slot's row is zeroed when it opens."""
        if name not in self._named_state:
            self._named_state[name] = torch.zeros((self.max_slots, *shape), dtype=dtype, device=self.device)
        return self._named_state[name]

    def kv_view(self, entry: int) -> ops.KVView:
        kind, g, i = self._entry_place[entry]
        if kind != "kv":
            raise KeyError(f"cache entry {entry} holds state, not keys and values")
        spec = self.kv_specs[g]
        return ops.KVView(self.kv_storage[g][i], self.block_tables[g], spec.n_kv, self.page_size, spec.head_dim)

    def state_view(self, entry: int) -> torch.Tensor:
        kind, g, i = self._entry_place[entry]
        if kind != "state":
            raise KeyError(f"cache entry {entry} holds keys and values, not state")
        return self.state_storage[g][i]

    # ------------------------------------------------------------------ slots

    def open(self, count: int = 1) -> List[int]:
        if count > self.book.slots.n_free:
            raise CacheFull(f"need {count} slots, {self.book.slots.n_free} of {self.max_slots} are free")
        slots = [self.book.open() for _ in range(count)]
        index = torch.tensor(slots, dtype=torch.int64, device=self.device)
        self.seq_lens.index_fill_(0, index, 0)
        for tensor in self._named_state.values():
            tensor.index_fill_(0, index, 0)
        for storage in self.state_storage:
            storage.index_fill_(1, index, 0)
        return slots

    def close(self, slots: Sequence[int]) -> None:
        updates: List[TableUpdate] = []
        for slot in slots:
            updates.extend(self.book.close(slot))
        self._apply(updates)

    def length(self, slot: int) -> int:
        return self.book.length(slot)

    # ------------------------------------------------------------------ steps

    def prepare(self, slots: Sequence[int], counts: Sequence[int]) -> None:
        """Map the pages that the step's new tokens will be written to."""
        self._apply(self.book.prepare(slots, counts))

    def commit(self, slots: Sequence[int], counts: Sequence[int]) -> None:
        """Record on the host that the step's tokens are in (the device lengths are advanced
        by the step itself) and release pages that fell out of a window."""
        self._apply(self.book.commit(slots, counts))

    def _apply(self, updates: Sequence[TableUpdate]) -> None:
        if not updates:
            return
        for g in range(len(self.kv_specs)):
            cells = [(slot * self.max_pages_per_seq + logical, physical)
                     for group, slot, logical, physical in updates if group == g]
            if not cells:
                continue
            packed = torch.tensor(cells, dtype=torch.int64).t().contiguous()
            index = packed[0].to(self.device, non_blocking=True)
            value = packed[1].to(torch.int32).to(self.device, non_blocking=True)
            ops.scatter_i32(self.block_tables[g], index, value)

    def tokens_held(self) -> int:
        return self.book.tokens_held()

    def check(self) -> None:
        self.book.check()
