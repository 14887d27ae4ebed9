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
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..cache.sequence_cache import SequenceCache
from ..parts import HostBatch, StepContext


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

    def run_rows(self, tokens: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor, n_rows: int,
                 max_q_len: int, max_context: Optional[int], want_rows: Optional[torch.Tensor],
                 inputs: Optional[Dict[str, torch.Tensor]] = None,
                 row_out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                 lengths_differ: Optional[bool] = None) -> Optional[torch.Tensor]:
        """The device side of a step, and the only forward pass there is: rows and positions
        from the sequences' lengths, the scheduled layers from the cache, final norm and head
        at ``want_rows`` (int32 row indices; None: every row; empty: none, returns None),
        lengths advanced.  Every argument lives on the device and nothing here synchronises,
        so the same call is recorded into the generation loop's decode graphs."""
        rows = ops.step_rows(cu_seqlens, slots, self.cache.seq_lens, n_rows, max_q_len, out=row_out,
                             max_context=max_context, lengths_differ=lengths_differ)
        ctx = StepContext(rows=rows, cache=self.cache, err=self.err, inputs=inputs or {})
        h, d = self.model.hidden(tokens, ctx)
        logits = None
        if want_rows is None or want_rows.shape[0]:
            logits = self.model.logits(h, d, want_rows, self.err)
        ops.advance(self.cache.seq_lens, slots, cu_seqlens)
        return logits

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
        held = [self.cache.length(slot) for slot in slots]

        # What parts want computed on the host for this step travels with the tokens.
        asked = self.model.step_inputs(HostBatch(slots, counts, held, self.cache.page_size))
        names = sorted(asked)
        parts = [[t for e in entries for t in e.tokens], cu, slots, want_rows] + [list(asked[n]) for n in names]
        packed = self._upload([x for part in parts for x in part])
        views, at = [], 0
        for part in parts:
            views.append(packed[at:at + len(part)])
            at += len(part)
        tokens, cu_dev, slots_dev, want_dev = views[:4]
        inputs = dict(zip(names, views[4:]))

        longest = max(h + c for h, c in zip(held, counts))
        logits = self.run_rows(tokens, cu_dev, slots_dev, n_rows, max(counts), longest, want_dev, inputs,
                               lengths_differ=ops.lengths_differ([h + c for h, c in zip(held, counts)]))
        if logits is None:
            logits = torch.empty((0, self.model.vocab_size), dtype=torch.float32, device=self.device)
        self.cache.commit(slots, counts)
        if check:
            ops.raise_on_device_error(self.err, "step")
        return logits
