"""Arrangement of a layer's parts.  ``pre_norm``: ``a = x + mixer(norm(x))``,
``y = a + ffn(norm(a))`` (OPTIMIZATION_GUIDE.md:57-70).  The add of a branch's output is
deferred to the next norm, which fuses it (engine/engine.py:1104-1118): a block takes and
returns the pair (residual stream ``h``, pending branch output ``d`` or None).

A block owns its sub-parts.  Their specs are parameters of the block's own spec, the block
builds them, lists their tensors, answers for their cache need and passes on what they
ask of a step.  The model above sees blocks only, so an arrangement with other members is
a new class of this family and nothing else.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..cache.sequence_cache import CacheNeed
from ..config.base import PartSpec, ScheduleEntry
from ..weights.loader import TensorSpec
from .registry import part_class, register_part
from .runtime import HostBatch, Runtime, StepContext


class Block:
    """Base of the block arrangements.  ``MEMBERS`` maps the names of the sub-part specs among
    the block's parameters to their families; a member whose spec is absent or None is left
    out (the attribute of that name is None)."""

    MEMBERS: Dict[str, str] = {}

    @classmethod
    def members(cls, spec: PartSpec) -> List[Tuple[str, str, PartSpec]]:
        return [(name, family, spec.params[name]) for name, family in cls.MEMBERS.items()
                if spec.params.get(name) is not None]

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        specs: List[TensorSpec] = []
        for _, family, member in cls.members(spec):
            specs += part_class(family, member.kind).tensor_specs(member)
        return specs

    def __init__(self, spec: PartSpec, runtime: Runtime):
        for name in self.MEMBERS:
            setattr(self, name, None)
        for name, family, member in self.members(spec):
            setattr(self, name, part_class(family, member.kind)(member, runtime))

    def parts(self) -> List[object]:
        return [getattr(self, name) for name in self.MEMBERS if getattr(self, name) is not None]

    def cache_need(self) -> CacheNeed:
        """What the block's cache entry stores: the need of its (one) mixer."""
        mixer = getattr(self, "mixer", None)
        return mixer.cache_need() if mixer is not None else None

    def step_inputs(self, batch: HostBatch, out: Dict[str, List[int]]) -> None:
        """Integer inputs that members want computed on the host for this step, by name."""
        for part in self.parts():
            if hasattr(part, "step_inputs"):
                part.step_inputs(batch, out)


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    MEMBERS = {"norm_mixer": "norm", "mixer": "mixer", "norm_ffn": "norm", "ffn": "ffn"}

    def forward(self, h: torch.Tensor, d: Optional[torch.Tensor], ctx: StepContext,
                entry: ScheduleEntry) -> Tuple[torch.Tensor, torch.Tensor]:
        n = self.norm_mixer.forward(h) if d is None else self.norm_mixer.add_forward(h, d)
        a = self.mixer.forward(n, ctx, entry)
        n = self.norm_ffn.add_forward(h, a)
        return h, self.ffn.forward(n, ctx)
