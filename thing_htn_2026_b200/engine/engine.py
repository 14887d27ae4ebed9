"""The Python entry point.  ``Engine(model_path).generate(input_ids, max_new_tokens)``
yields one token id per sequence per step, exactly ``max_new_tokens`` times, and never
stops at an end-of-sequence token unless told to: the reference's interface
(README.md:48-66; engine/engine.py:109-111, :1225-1230).  Beyond it: prompts of unequal
lengths, temperature and seed, stop tokens, a queue of requests run as successive batches,
and a random-weights constructor.

Environment switches keep the reference's names and meanings: ``DRYFT_ENGINE_GRAPHS``
(CUDA graphs for decode steps, default on) and ``DRYFT_ENGINE_DEPTH`` (decode steps in
flight ahead of the host, default 3) (engine/engine.py:121-123).
"""

from __future__ import annotations

import os
from typing import Iterator, List, Optional, Sequence

import torch

from ..cache.sequence_cache import SequenceCache
from ..config import ModelConfig
from .device_backend import DeviceBackend
from .generation import Completion, GenerationLoop, Request, tokens_needed
from .loading import load_model, parse_dtype, random_model


def _env_flag(name: str, default: bool) -> bool:
    value = os.environ.get(name)
    if value is None:
        return default
    return value.strip().lower() not in ("0", "false", "no", "off", "")


class Engine:
    def __init__(self, model_path: Optional[str] = None, *, dtype="bfloat16", device: str = "cuda:0",
                 max_tokens: Optional[int] = None, max_batch: int = 64, graphs: Optional[bool] = None,
                 depth: Optional[int] = None, model=None) -> None:
        """Loads the checkpoint of ``model_path`` (config.json + safetensors).  ``max_tokens``
        fixes the size of the cache; left out, the cache is sized by the first call that
        needs more (as the reference sizes its cache per shape, engine/engine.py:830-846)."""
        if not torch.cuda.is_available():
            raise RuntimeError("Engine needs a CUDA device; this library has no CPU path")
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        self.model = model if model is not None else load_model(model_path, self.dtype, device)
        self.use_graphs = _env_flag("DRYFT_ENGINE_GRAPHS", True) if graphs is None else bool(graphs)
        self.depth = max(1, int(os.environ.get("DRYFT_ENGINE_DEPTH", 3) if depth is None else depth))
        self.max_batch = int(max_batch)
        self.backend: Optional[DeviceBackend] = None
        self.loop: Optional[GenerationLoop] = None
        self._fixed_tokens = max_tokens
        if max_tokens is not None:
            self._build_cache(int(max_tokens))

    @classmethod
    def from_config(cls, config: ModelConfig, seed: int = 0, *, dtype="bfloat16", device: str = "cuda:0",
                    matrix_std: float = 0.02, gain_std: float = 0.02, **kwargs) -> "Engine":
        """Random weights of the configuration's shapes, drawn on the device."""
        model = random_model(config, seed, dtype, device, matrix_std=matrix_std, gain_std=gain_std)
        return cls(None, dtype=dtype, device=device, model=model, **kwargs)

    # ------------------------------------------------------------------ cache

    def _build_cache(self, max_tokens: int) -> None:
        self.backend = None
        self.loop = None
        page = 64
        pages = -(-max_tokens // page) + 1          # one page for the backend's scratch slot
        cache = SequenceCache(self.model.cache_needs(), max_tokens=pages * page, dtype=self.dtype,
                              device=self.device, max_slots=max(2, min(pages, self.max_batch + 1)))
        self.backend = DeviceBackend(self.model, cache, max_batch=self.max_batch, use_graphs=self.use_graphs,
                                     ring=self.depth + 2)
        self.loop = GenerationLoop(self.backend, self.depth)

    def _ensure_cache(self, requests: Sequence[Request], whole_queue_in_one_batch: bool) -> None:
        page = 64
        if whole_queue_in_one_batch:
            need = sum(tokens_needed(r, page) for r in requests)
        else:
            need = max(tokens_needed(r, page) for r in requests)
        if self.backend is not None and need <= self.backend.capacity_tokens():
            return
        if self._fixed_tokens is not None:
            raise ValueError(f"the batch needs {need} cache tokens, the engine was built with "
                             f"max_tokens={self._fixed_tokens}")
        self._build_cache(need)

    # ------------------------------------------------------------------ generation

    def _requests(self, input_ids, max_new_tokens, temperature, seed, stop_token_ids) -> List[Request]:
        n = len(input_ids)
        limits = list(max_new_tokens) if isinstance(max_new_tokens, (list, tuple)) else [int(max_new_tokens)] * n
        temps = list(temperature) if isinstance(temperature, (list, tuple)) else [float(temperature)] * n
        if len(limits) != n or len(temps) != n:
            raise ValueError("per-sequence max_new_tokens and temperature must have one entry per sequence")
        vocab = self.model.vocab_size
        for i, ids in enumerate(input_ids):
            for t in ids:
                if not 0 <= int(t) < vocab:
                    raise ValueError(f"sequence {i}: token id {t} is outside the vocabulary [0, {vocab})")
        return [Request(list(ids), limits[i], temps[i], int(seed), i, tuple(stop_token_ids or ()))
                for i, ids in enumerate(input_ids)]

    def generate(self, input_ids: Sequence[Sequence[int]], max_new_tokens, *, temperature=0.0, seed: int = 0,
                 stop_token_ids: Optional[Sequence[int]] = None) -> Iterator[List[Optional[int]]]:
        """Continues every sequence one step at a time, as one batch.  Yields a list with
        one token id per sequence per output step.  Without stop tokens and with one
        ``max_new_tokens`` for all, that is exactly ``max_new_tokens`` lists of ints.  A
        sequence that has finished (its stop token or its own limit) yields None from then
        on; generation ends when all have finished."""
        requests = self._requests(input_ids, max_new_tokens, temperature, seed, stop_token_ids)
        if not requests or max(r.max_new_tokens for r in requests) <= 0:
            return
        if len(requests) > self.max_batch:
            raise ValueError(f"{len(requests)} sequences exceed max_batch={self.max_batch}; "
                             f"use generate_all for a queue of requests")
        self._ensure_cache(requests, whole_queue_in_one_batch=True)
        with torch.inference_mode():
            yield from self.loop.run_batch(requests)

    def generate_all(self, input_ids: Sequence[Sequence[int]], max_new_tokens, *, temperature=0.0, seed: int = 0,
                     stop_token_ids: Optional[Sequence[int]] = None) -> List[Completion]:
        """Any number of requests, run as successive batches that fit the cache and
        ``max_batch``.  Returns one Completion (tokens, finish_reason) per request."""
        requests = self._requests(input_ids, max_new_tokens, temperature, seed, stop_token_ids)
        if not requests:
            return []
        self._ensure_cache(requests, whole_queue_in_one_batch=len(requests) <= self.max_batch)
        with torch.inference_mode():
            return self.loop.generate_all(requests)
