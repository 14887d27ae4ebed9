"""Token choice.  Greedy (the reference's only mode, engine/engine.py:1121) and
temperature sampling; both run on the device (csrc/sampling.cu) on float32 logits.

``temperature == 0`` is greedy: argmax, lowest index on exact ties.  ``temperature > 0``
draws from ``softmax(logits / temperature)`` by the Gumbel-max rule with counter-based
noise: the draw of a sequence at its n-th generated token depends only on
``(seed, stream, n)``, where ``stream`` is the request's index unless given, so a
sequence samples the same tokens alone or in any batch.

:class:`TokenChooser` keeps what the choice needs as per-sequence state of fixed size in
the cache, indexed by slot: temperature, seed, stream, the count of tokens drawn so far,
and the token chosen last (which the next single-token step feeds back without a visit to
the host).
"""

from __future__ import annotations

from typing import Sequence

import torch

from .. import ops


def as_int64(seed: int) -> int:
    """Any Python integer seed as the signed 64-bit value of its low 64 bits."""
    seed &= 0xFFFFFFFFFFFFFFFF
    return seed - (1 << 64) if seed >= (1 << 63) else seed


class TokenChooser:
    def __init__(self, cache):
        state = cache.sequence_state
        self.device = cache.device
        self.last_token = state("last_token", (), torch.int32)
        self.sample_step = state("sample_step", (), torch.int32)
        self.temperature = state("temperature", (), torch.float32)
        self.seed = state("seed", (), torch.int64)
        self.stream_id = state("stream", (), torch.int32)

    def configure(self, slots: Sequence[int], temperatures: Sequence[float], seeds: Sequence[int],
                  streams: Sequence[int]) -> None:
        """Sets the sampling state of freshly opened slots (their draw counters are zero)."""
        index = torch.tensor(list(slots), dtype=torch.int64, device=self.device)
        self.temperature.index_copy_(0, index, torch.tensor(list(temperatures), dtype=torch.float32,
                                                            device=self.device))
        self.seed.index_copy_(0, index, torch.tensor([as_int64(s) for s in seeds], dtype=torch.int64,
                                                     device=self.device))
        self.stream_id.index_copy_(0, index, torch.tensor([s & 0x7FFFFFFF for s in streams], dtype=torch.int32,
                                                          device=self.device))

    def choose(self, logits: torch.Tensor, slots: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """One token per row of ``logits`` (float32 ``[rows, vocab]``) for the sequences in
        ``slots`` (int32, on the device): written to ``out`` and to each sequence's
        ``last_token``; its draw counter goes up by one."""
        return ops.choose_tokens(logits, self.temperature, self.seed, self.stream_id, self.sample_step, out=out,
                                 slots=slots, last_token=self.last_token, bump_step=True)


def greedy(logits: torch.Tensor) -> torch.Tensor:
    """float32 [rows, vocab] on the device -> int32 [rows]: argmax, lowest index on ties."""
    return ops.choose_tokens(logits)


__all__ = ["TokenChooser", "as_int64", "greedy"]
