"""Device side of the generation loop: prefill through the step function, single-token
steps as one CUDA graph per batch size and class of context length, token choice on the device, tokens back to the
host through a ring of pinned buffers.

Per-sequence state of fixed size, indexed by slot (beside ``seq_lens``): the token the
sequence feeds next, its sampling step counter, temperature, seed and stream.  A decode
step reads its batch as a list of slots from a static buffer, so one captured graph
serves every batch of that size; the next token never visits the host before it is fed
back.  (The reference keeps a token history and positions on the device for the same
reason, engine/engine.py:941-953, and captures the step once per shape, :1005-1042.)
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..cache.sequence_cache import SequenceCache
from ..parts import StepContext
from ..sampling import TokenChooser
from .generation import Request, tokens_needed
from .step import StepEntry, StepRunner


@dataclass
class _Handle:
    buffer: torch.Tensor     # pinned int32
    event: torch.cuda.Event
    count: int
    place: int               # in the ring


class DeviceBackend:
    def __init__(self, model, cache: SequenceCache, *, max_batch: int = 64, use_graphs: bool = True,
                 ring: int = 8):
        """``ring``: pinned token buffers for steps whose tokens the host has not fetched yet;
        a generation loop of depth d keeps d + 1 such steps, so it needs ``ring >= d + 1``.
        Sending one more than the ring holds raises instead of overwriting."""
        self.model, self.cache = model, cache
        self.device = model.device
        self.page_size = cache.page_size
        self._max_batch = min(int(max_batch), cache.max_slots - 1)
        self.use_graphs = bool(use_graphs)
        self.runner = StepRunner(model, cache)
        self.err = self.runner.err
        self.chooser = TokenChooser(cache)
        self.last_token = self.chooser.last_token

        n = self._max_batch
        dev = self.device
        self.slots_buf = torch.zeros(n, dtype=torch.int32, device=dev)
        self.cu_buf = torch.arange(n + 1, dtype=torch.int32, device=dev)
        self.tokens_in = torch.zeros(n, dtype=torch.int32, device=dev)
        self.out_tokens = torch.zeros(n, dtype=torch.int32, device=dev)
        self.row_slot = torch.zeros(n, dtype=torch.int32, device=dev)
        self.row_pos = torch.zeros(n, dtype=torch.int32, device=dev)
        self.graphs: Dict[Tuple[int, int, bool], torch.cuda.CUDAGraph] = {}     # (batch, context class, lengths differ)
        self._composition: Optional[Tuple[int, ...]] = None
        ring = max(2, int(ring))
        self._ring = [(torch.zeros(max(n, 1), dtype=torch.int32, pin_memory=True), torch.cuda.Event())
                      for _ in range(ring)]
        self._ring_busy = [False] * ring          # sent and not fetched yet
        self._stage = [torch.zeros(max(n, 1), dtype=torch.int32, pin_memory=True) for _ in range(ring)]
        self._ring_next = 0
        self.graph_logits: Dict[Tuple[int, int, bool], torch.Tensor] = {}    # the captured programs' logits
        # One slot with one page stays reserved: decode graphs are warmed up on it.
        (self._scratch_slot,) = cache.open(1)
        cache.prepare([self._scratch_slot], [1])
        self.kernel_launches = 0

    # ------------------------------------------------------------------ capacity

    def capacity_tokens(self) -> int:
        return (self.cache.n_pages - 1) * self.page_size

    def max_batch(self) -> int:
        return self._max_batch

    # ------------------------------------------------------------------ batches

    def open_batch(self, requests: Sequence[Request]) -> List[int]:
        # Pages are mapped step by step: the prompt's here, a new one whenever a sequence crosses
        # a page boundary (launch_decode).  A batch is admitted by its full length
        # (generation.form_batches) and batches run one at a time, so the pages are there when
        # they are asked for; a windowed group meanwhile gives pages back and maps them again.
        slots = self.cache.open(len(requests))
        try:
            self.cache.prepare(slots, [len(r.tokens) for r in requests])
        except Exception:
            self.cache.close(slots)
            raise
        self.chooser.configure(slots, [r.temperature for r in requests], [r.seed for r in requests],
                               [r.stream for r in requests])
        self._composition = None
        return slots

    def close_batch(self, slots: Sequence[int]) -> None:
        self.cache.close(slots)
        ops.raise_on_device_error(self.err, "generation")      # reads the error word: every step has ended
        self._ring_busy = [False] * len(self._ring)            # handles of an abandoned batch are void

    # ------------------------------------------------------------------ steps

    def _send(self, tokens_dev: torch.Tensor, count: int) -> _Handle:
        at = self._ring_next
        if self._ring_busy[at]:
            raise RuntimeError(f"{len(self._ring) + 1} steps are in flight whose tokens the host has not fetched; "
                               f"the backend was built with a ring of {len(self._ring)}")
        buffer, event = self._ring[at]
        self._ring_next = (at + 1) % len(self._ring)
        self._ring_busy[at] = True
        buffer[:count].copy_(tokens_dev[:count], non_blocking=True)
        event.record()
        return _Handle(buffer, event, count, at)

    def launch_prefill(self, slots: Sequence[int], prompts: Sequence[Sequence[int]]) -> _Handle:
        entries = [StepEntry(slot, prompt, (len(prompt) - 1,)) for slot, prompt in zip(slots, prompts)]
        logits = self.runner.step(entries, check=False)
        slots_dev = self.runner._upload(list(slots))
        out = torch.empty(len(slots), dtype=torch.int32, device=self.device)
        self.chooser.choose(logits, slots_dev, out)
        return self._send(out, len(slots))

    def _decode_program(self, batch: int, max_context: int, lengths_differ: Optional[bool] = None) -> torch.Tensor:
        """One token for each of the first ``batch`` slots of ``slots_buf``: the step function's
        device side (``StepRunner.run_rows``) between a gather of each sequence's last token
        and the token choice.  Everything it reads and writes is per-sequence state or a
        static buffer.  ``max_context`` bounds the keys a sequence holds after the step, for
        as long as the program is replayed.  Returns the step's logits."""
        slots = self.slots_buf[:batch]
        tokens = ops.gather_i32(self.last_token, slots, out=self.tokens_in[:batch])
        logits = self.runner.run_rows(tokens, self.cu_buf[:batch + 1], slots, batch, 1, max_context, None,
                                      row_out=(self.row_slot[:batch], self.row_pos[:batch]),
                                      lengths_differ=lengths_differ)
        self.chooser.choose(logits, slots, self.out_tokens[:batch])
        return logits

    def _set_composition(self, slots: Sequence[int]) -> None:
        key = tuple(slots)
        if key == self._composition:
            return
        stage = self._stage[self._ring_next]
        stage[:len(slots)] = torch.tensor(list(slots), dtype=torch.int32)
        self.slots_buf[:len(slots)].copy_(stage[:len(slots)], non_blocking=True)
        self._composition = key

    def _capture(self, batch: int, context_class: int, max_context: int, differ: bool) -> None:
        """Warm the program up on the scratch slot (it advances nothing that lives), then
        record it."""
        scratch = torch.full((batch,), self._scratch_slot, dtype=torch.int32, device=self.device)
        self.slots_buf[:batch].copy_(scratch)
        self._composition = None
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self.cache.seq_lens[self._scratch_slot] = 0
                self._decode_program(batch, max_context, differ)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.graph_logits[(batch, context_class, differ)] = self._decode_program(batch, max_context, differ)
        self.cache.seq_lens[self._scratch_slot] = 0
        torch.cuda.synchronize()
        self.graphs[(batch, context_class, differ)] = graph

    def launch_decode(self, slots: Sequence[int]) -> _Handle:
        batch = len(slots)
        lengths = [self.cache.length(slot) + 1 for slot in slots]
        context_class, max_context = ops.context_class(max(lengths))
        differ = ops.lengths_differ(lengths)
        if self.use_graphs and (batch, context_class, differ) not in self.graphs:
            self._capture(batch, context_class, max_context, differ)
        self.cache.prepare(list(slots), [1] * batch)          # a block-table update only at page boundaries
        self._set_composition(slots)
        if self.use_graphs:
            self.graphs[(batch, context_class, differ)].replay()
        else:
            self._decode_program(batch, max_context, differ)
        self.cache.commit(list(slots), [1] * batch)
        return self._send(self.out_tokens, batch)

    def fetch(self, handle: _Handle) -> List[int]:
        handle.event.synchronize()
        tokens = handle.buffer[:handle.count].tolist()
        self._ring_busy[handle.place] = False
        return tokens
