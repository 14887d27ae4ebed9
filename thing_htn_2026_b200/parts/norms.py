"""RMSNorm.  ``forward`` normalises; ``add_forward`` first adds a branch's output to the
residual stream in place (the reference fuses the two the same way,
engine/kernels/torch_ref.py:61-68, engine/engine.py:1104-1107)."""

from __future__ import annotations

from typing import List

import torch

from .. import ops
from ..config.base import PartSpec
from ..weights.loader import GAIN, TensorSpec
from .registry import register_part
from .runtime import Runtime


@register_part("norm", "rmsnorm")
class RMSNorm:
    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        return [TensorSpec(spec.tensors["weight"], (int(spec.params["size"]),), GAIN)]

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.gain = runtime.tensor(spec, "weight")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.gain, self.eps)

    def add_forward(self, h: torch.Tensor, d: torch.Tensor) -> torch.Tensor:
        return ops.add_rmsnorm(h, d, self.gain, self.eps)
