"""Token choice.  Greedy (the reference's only mode, engine/engine.py:1121) and
temperature sampling; both run on the device (csrc/sampling.cu) on float32 logits.

``temperature == 0`` is greedy: argmax, lowest index on exact ties.  ``temperature > 0``
draws from ``softmax(logits / temperature)`` by the Gumbel-max rule with counter-based
noise: the draw of a sequence at its n-th generated token depends only on
``(seed, stream, n)``, where ``stream`` is the request's index unless given, so a
sequence samples the same tokens alone or in any batch.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .. import ops


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0
    stream: Optional[int] = None
    stop_token_ids: Tuple[int, ...] = ()


def greedy(logits: torch.Tensor) -> torch.Tensor:
    """float32 [rows, vocab] on the device -> int32 [rows]."""
    return ops.choose_tokens(logits)


def sample(logits: torch.Tensor, temperature: torch.Tensor, seed: torch.Tensor, stream: torch.Tensor,
           step: torch.Tensor) -> torch.Tensor:
    """Per-row temperature (float32), seed (int64), stream and step (int32), all on the device."""
    return ops.choose_tokens(logits, temperature, seed, stream, step)
