"""Token embedding (a row gather, engine/engine.py:1101) and the LM head
(engine/engine.py:1120; with tied weights it is the embedding table, :225-226).
Logits are float32."""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from ..config.base import PartSpec
from ..weights.loader import MATRIX, TensorSpec
from .registry import register_part
from .runtime import Runtime


@register_part("embedding", "embedding")
class Embedding:
    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        return [TensorSpec(spec.tensors["weight"], (int(spec.params["vocab_size"]), int(spec.params["hidden_size"])),
                           MATRIX)]

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.table = runtime.tensor(spec, "weight")

    def forward(self, tokens: torch.Tensor, err: torch.Tensor) -> torch.Tensor:
        return ops.gather_rows(self.table, tokens, err)


@register_part("head", "lm_head")
class LMHead:
    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        copies = (spec.tensors["stored_copy"],) if "stored_copy" in spec.tensors else ()
        return [TensorSpec(spec.tensors["weight"], (int(spec.params["vocab_size"]), int(spec.params["hidden_size"])),
                           MATRIX, copies=copies)]

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.weight = runtime.tensor(spec, "weight")
        self.vocab_size = int(spec.params["vocab_size"])

    def forward(self, x: torch.Tensor, err: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.linear(x, self.weight, out_dtype=torch.float32, err=err)
