"""What a part gets from its surroundings: at construction the precision, the device and
its tensors; at every step the rows, the cache and the error word."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional

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


@dataclass
class StepContext:
    """Step-time surroundings of a part.  ``rows`` says, for each packed row, which slot it
    belongs to and its position; ``cache`` holds keys, values and per-sequence state."""

    rows: ops.StepRows
    cache: "object"
    err: torch.Tensor
    extras: Dict[str, object] = field(default_factory=dict)
