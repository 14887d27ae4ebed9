"""The generation loop: host-side decisions only.  It forms batches from a queue of
requests, starts a batch with one prefill step over unequal prompts, then launches
single-token steps for the sequences that still need tokens, keeps a few steps in flight,
stops sequences at their stop tokens or their own token limit, and gives the batch's
slots back when it ends.  All device work is behind a small backend interface, so the
decisions can be tested without a device.

The reference's loop (engine/engine.py:1225-1250, :1309-1380) runs equal prompts for a
fixed count, never stops at a token (README.md:64), keeps ``pipeline_depth`` graph
replays in flight (:1254-1288) and never launches a step that cannot be needed
(:1332-1336; tests/launch_count.py:57-65).  The same rule holds here: with no stop
tokens a batch launches exactly ``max(max_new_tokens) - 1`` decode steps.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Iterator, List, Optional, Protocol, Sequence, Tuple

PAGE_ROUND = 64


@dataclass
class Request:
    tokens: Sequence[int]
    max_new_tokens: int
    temperature: float = 0.0
    seed: int = 0
    stream: int = 0                    # distinguishes requests that share a seed
    stop_token_ids: Tuple[int, ...] = ()

    def __post_init__(self):
        if len(self.tokens) == 0:
            raise ValueError("a request needs at least one prompt token")
        if self.max_new_tokens < 0:
            raise ValueError(f"max_new_tokens must not be negative, got {self.max_new_tokens}")
        if self.temperature < 0:
            raise ValueError(f"temperature must not be negative, got {self.temperature}")
        self.stop_token_ids = tuple(int(t) for t in (self.stop_token_ids or ()))


@dataclass
class Completion:
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""            # "length" or "stop"


class Backend(Protocol):
    page_size: int

    def capacity_tokens(self) -> int: ...
    def max_batch(self) -> int: ...
    def open_batch(self, requests: Sequence[Request]) -> List[int]: ...
    def launch_prefill(self, slots: Sequence[int], prompts: Sequence[Sequence[int]]) -> object: ...
    def launch_decode(self, slots: Sequence[int]) -> object: ...
    def fetch(self, handle: object) -> List[int]: ...
    def close_batch(self, slots: Sequence[int]) -> None: ...


def tokens_needed(request: Request, page_size: int) -> int:
    """Cache tokens a request can come to hold, rounded up to whole pages.  The last
    generated token is never fed back, so it needs no place."""
    n = len(request.tokens) + max(0, request.max_new_tokens - 1)
    return -(-n // page_size) * page_size


def form_batches(requests: Sequence[Request], capacity_tokens: int, max_batch: int, page_size: int) -> List[List[int]]:
    """Splits the queue, in order, into batches that fit the cache and the batch limit.
    Returns lists of request indices."""
    batches: List[List[int]] = []
    current: List[int] = []
    used = 0
    for i, request in enumerate(requests):
        need = tokens_needed(request, page_size)
        if need > capacity_tokens:
            raise ValueError(
                f"request {i} needs {need} cache tokens (prompt {len(request.tokens)} + "
                f"{request.max_new_tokens} new), the cache holds {capacity_tokens}")
        if current and (len(current) >= max_batch or used + need > capacity_tokens):
            batches.append(current)
            current, used = [], 0
        current.append(i)
        used += need
    if current:
        batches.append(current)
    return batches


class GenerationLoop:
    def __init__(self, backend: Backend, depth: int = 3):
        self.backend = backend
        self.depth = max(1, int(depth))
        self.decode_launches = 0       # of the last batch; the over-launch rule is tested on it

    def run_batch(self, requests: Sequence[Request],
                  completions: Optional[List[Completion]] = None) -> Iterator[List[Optional[int]]]:
        """One batch from start to end.  Yields, per output step, one entry per request: the
        token, or None once that request has finished.  Ends when all have finished.  If
        ``completions`` is given, tokens and finish reasons are also collected there."""
        n = len(requests)
        limits = [r.max_new_tokens for r in requests]
        self.decode_launches = 0
        if n == 0 or max(limits) == 0:
            return
        if completions is None:
            completions = [Completion() for _ in requests]
        backend = self.backend
        slots = backend.open_batch(requests)
        try:
            finished = [limit == 0 for limit in limits]
            launched = [0] * n          # tokens whose computation has been launched, per request
            produced = [0] * n          # tokens seen by the host, per request
            inflight: Deque[Tuple[object, List[int]]] = deque()

            starters = [i for i in range(n) if not finished[i]]
            inflight.append((backend.launch_prefill([slots[i] for i in starters],
                                                    [requests[i].tokens for i in starters]), starters))
            for i in starters:
                launched[i] += 1

            while inflight:
                while len(inflight) <= self.depth:
                    members = [i for i in range(n) if not finished[i] and launched[i] < limits[i]]
                    if not members:
                        break
                    inflight.append((backend.launch_decode([slots[i] for i in members]), members))
                    self.decode_launches += 1
                    for i in members:
                        launched[i] += 1
                handle, members = inflight.popleft()
                tokens = backend.fetch(handle)
                out: List[Optional[int]] = [None] * n
                for i, token in zip(members, tokens):
                    if finished[i]:
                        continue           # launched before the host saw its stop token
                    token = int(token)
                    out[i] = token
                    produced[i] += 1
                    completions[i].tokens.append(token)
                    if token in requests[i].stop_token_ids:
                        finished[i], completions[i].finish_reason = True, "stop"
                    elif produced[i] >= limits[i]:
                        finished[i], completions[i].finish_reason = True, "length"
                if any(t is not None for t in out):
                    yield out
        finally:
            backend.close_batch(slots)

    def generate_all(self, requests: Sequence[Request]) -> List[Completion]:
        """As many batches, one after another, as the requests need."""
        completions = [Completion() for _ in requests]
        order = form_batches(requests, self.backend.capacity_tokens(), self.backend.max_batch(),
                             self.backend.page_size)
        self.batches_run = order
        for members in order:
            batch = [requests[i] for i in members]
            collected = [completions[i] for i in members]
            for _ in self.run_batch(batch, collected):
                pass
        for c, r in zip(completions, requests):
            if not c.finish_reason:
                c.finish_reason = "length"
        return completions
