"""What a part gets from its surroundings: at construction the precision, the device and
its tensors; at every step the rows, the cache and the error word."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
from ..config.base import PartSpec, ScheduleEntry


@dataclass
class Runtime:
    """Construction-time surroundings of a part."""

    dtype: torch.dtype
    device: torch.device
    tensors: Dict[str, torch.Tensor]
    shared: Dict[str, object] = field(default_factory=dict)   # parts built once per model, by PartSpec.key()

    def tensor(self, spec: PartSpec, name: str) -> torch.Tensor:
        return self.tensors[spec.tensors[name]]


@dataclass(frozen=True)
class HostBatch:
    """What the host knows of a step before it runs: for each sequence its slot, the tokens
    it brings and the tokens it already holds, in the order of the packed rows."""

    slots: Sequence[int]
    counts: Sequence[int]
    held: Sequence[int]
    page_size: int

    @property
    def row_starts(self) -> List[int]:
        starts, at = [], 0
        for c in self.counts:
            starts.append(at)
            at += c
        return starts

    @property
    def max_count(self) -> int:
        return max(self.counts) if self.counts else 0


@dataclass
class StepContext:
    """Step-time surroundings of a part.  ``rows`` says, for each packed row, which slot it
    belongs to and its position; ``cache`` holds keys, values and per-sequence state;
    ``inputs`` holds, by name, the int32 device tensors that parts asked for through
    ``step_inputs`` (they travel in the step's one upload)."""

    rows: ops.StepRows
    cache: "object"
    err: torch.Tensor
    inputs: Dict[str, torch.Tensor] = field(default_factory=dict)
    extras: Dict[str, object] = field(default_factory=dict)
