"""Dense feed-forward with a gated SiLU: ``down(silu(gate(x)) * up(x))``.  Gate and up
are one product over the concatenated weight ``[2I, H]`` (engine/engine.py:221, :1116-1118);
the activation rounds as engine/kernels/torch_ref.py:74-88 does."""

from __future__ import annotations

from typing import List

import torch

from .. import ops
from ..config.base import PartSpec
from ..weights.loader import MATRIX, TensorSpec
from .registry import register_part
from .runtime import Runtime


@register_part("ffn", "swiglu")
class SwiGLU:
    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        hidden, inter = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        return [TensorSpec(spec.tensors["gate_proj"], (inter, hidden), MATRIX),
                TensorSpec(spec.tensors["up_proj"], (inter, hidden), MATRIX),
                TensorSpec(spec.tensors["down_proj"], (hidden, inter), MATRIX)]

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.w_gate_up = torch.cat([runtime.tensor(spec, "gate_proj"), runtime.tensor(spec, "up_proj")], dim=0).contiguous()
        self.w_down = runtime.tensor(spec, "down_proj")

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        err = getattr(ctx, "err", None)
        return ops.linear(ops.linear_swiglu(x, self.w_gate_up, err), self.w_down, err=err)
