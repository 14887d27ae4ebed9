"""Rotary position encoding: the angle tables.  The rotation itself is fused into the
kernel that normalises q and k and writes the cache.

``inv_freq[i] = 1 / theta^(2i / rotary_dim)`` is computed once on the host in float32 with
the reference's expression (engine/engine.py:238-240); the device fills
``cos/sin[p, i]`` of ``p * inv_freq[i]`` in float32 (engine/engine.py:241-247).  The
tables cover the longest sequence of the cache and grow on demand (the reference grows
its tables the same way, engine/engine.py:232-251)."""

from __future__ import annotations

from typing import List

import torch

from .. import ops
from ..config.base import PartSpec
from ..weights.loader import TensorSpec
from .registry import register_part
from .runtime import Runtime


@register_part("position", "rope")
class Rope:
    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        return []

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.head_dim = int(spec.params["head_dim"])
        self.rotary_dim = int(spec.params.get("rotary_dim", self.head_dim))
        self.theta = float(spec.params["theta"])
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rope: rotary_dim {self.rotary_dim} must be even and within head_dim {self.head_dim}")
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.int64).to(torch.float32) / self.rotary_dim
        self.inv_freq = (1.0 / (self.theta ** exponent)).to(runtime.device)
        self.device = runtime.device
        self._tables = None

    def ensure(self, n_positions: int) -> None:
        """Tables for positions ``[0, n_positions)``.  Call before a CUDA graph is captured."""
        have = 0 if self._tables is None else self._tables.cos.shape[0]
        if n_positions <= have:
            return
        size = max(64, 1 << (int(n_positions) - 1).bit_length())
        half = self.rotary_dim // 2
        cos = torch.empty((size, half), dtype=torch.float32, device=self.device)
        sin = torch.empty((size, half), dtype=torch.float32, device=self.device)
        ops.rope_table(cos, sin, self.inv_freq, 0, size)
        self._tables = ops.RotaryTables(cos, sin, self.rotary_dim)

    def tables(self) -> ops.RotaryTables:
        if self._tables is None:
            raise RuntimeError("rope: ensure(n_positions) has not been called")
        return self._tables
