"""The step function: one batch of sequences, the tokens it brings, logits where wanted.

A step runs only the tokens it is given, as one packed batch ``[sum of lengths]`` with no
padding, on top of what earlier steps left in the cache.  The sequences of a step either
all start (prompts of unequal lengths, one step) or all go on by one token; the kernels
make no such distinction: every row carries its slot and its absolute position.

The reference has two functions with equal lengths only: ``_prefill_slice`` for prompts
(engine/engine.py:1191-1221) and ``_step`` for T tokens per sequence
(engine/engine.py:1093-1121); both return token ids, never logits.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from .. import ops
from ..cache.sequence_cache import SequenceCache
from ..parts import StepContext


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()     # places among ``tokens`` whose logits are asked for


class StepRunner:
    """Owns the device error word and drives ``model`` over ``cache``."""

    def __init__(self, model, cache: SequenceCache):
        self.model = model
        self.cache = cache
        self.device = model.device
        self.err = ops.new_error_word(self.device)
        model.ensure_positions(cache.max_pages_per_seq * cache.page_size)
        # Host-to-device uploads go through a small ring of pinned buffers; a buffer is reused
        # only after the copy that read it has finished.
        self._staging = [[None, None] for _ in range(4)]     # [pinned int32 tensor, event]
        self._staging_next = 0
        self.uploaded_bytes = 0

    def _upload(self, values: List[int]) -> torch.Tensor:
        """One asynchronous copy of ``values`` (int32) from pinned host memory."""
        slot = self._staging[self._staging_next]
        self._staging_next = (self._staging_next + 1) % len(self._staging)
        n = len(values)
        if slot[0] is None or slot[0].numel() < n:
            slot[0] = torch.empty(max(1024, 2 * n), dtype=torch.int32, pin_memory=True)
            slot[1] = torch.cuda.Event()
        else:
            slot[1].synchronize()
        slot[0].numpy()[:n] = values          # through numpy: the buffer may have been made in inference mode
        device = slot[0][:n].to(self.device, non_blocking=True)
        slot[1].record()
        self.uploaded_bytes += 4 * n
        return device

    def step(self, entries: Sequence[StepEntry], check: bool = True) -> torch.Tensor:
        """Runs the entries' tokens; returns float32 logits ``[wanted, vocab]`` in the order
        of the entries and of their ``want``.  Raises CacheFull before touching anything if
        the cache cannot take the tokens."""
        entries = [e for e in entries]
        slots = [e.slot for e in entries]
        counts = [len(e.tokens) for e in entries]
        if any(c == 0 for c in counts):
            raise ValueError("a step entry brings no tokens")
        n_rows = sum(counts)
        cu = [0]
        for c in counts:
            cu.append(cu[-1] + c)
        want_rows: List[int] = []
        for e, start in zip(entries, cu):
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise ValueError(f"slot {e.slot}: wanted place {w} is outside its {len(e.tokens)} tokens")
                want_rows.append(start + w)
        self.cache.prepare(slots, counts)

        tile_row0: List[int] = []
        tile_rows: List[int] = []
        if max(counts) > 1:
            # Row tiles for the prompt attention kernels, the ones that see the fewest keys
            # first: the kernels start at the end of the list, so the longest run first and
            # the short ones fill the gaps at the end.
            size = ops.ROW_TILE()
            tiles = []
            for slot, start, c in zip(slots, cu, counts):
                held = self.cache.length(slot)
                for r in range(0, c, size):
                    n = min(size, c - r)
                    tiles.append((held + r + n, start + r, n))
            tiles.sort()
            tile_row0 = [t[1] for t in tiles]
            tile_rows = [t[2] for t in tiles]

        parts = [[t for e in entries for t in e.tokens], cu, slots, want_rows, tile_row0, tile_rows]
        packed = self._upload([x for part in parts for x in part])
        views, at = [], 0
        for part in parts:
            views.append(packed[at:at + len(part)])
            at += len(part)
        tokens, cu_dev, slots_dev, want_dev, tile_row0_dev, tile_rows_dev = views

        longest = max(self.cache.length(slot) + c for slot, c in zip(slots, counts))
        rows = ops.step_rows(cu_dev, slots_dev, self.cache.seq_lens, n_rows, max(counts), max_context=longest)
        if tile_row0:
            rows.tile_row0, rows.tile_rows, rows.n_tiles = tile_row0_dev, tile_rows_dev, len(tile_row0)
        ctx = StepContext(rows=rows, cache=self.cache, err=self.err)
        h, d = self.model.hidden(tokens, ctx)
        if want_rows:
            logits = self.model.logits(h, d, want_dev, self.err)
        else:
            logits = torch.empty((0, self.model.vocab_size), dtype=torch.float32, device=self.device)
        ops.advance(self.cache.seq_lens, slots_dev, cu_dev)
        self.cache.commit(slots, counts)
        if check:
            ops.raise_on_device_error(self.err, "step")
        return logits
