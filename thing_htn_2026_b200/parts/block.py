"""Arrangement of a layer's parts.  ``pre_norm``: ``a = x + mixer(norm(x))``,
``y = a + ffn(norm(a))`` (OPTIMIZATION_GUIDE.md:57-70).  The add of a branch's output is
deferred to the next norm, which fuses it (engine/engine.py:1104-1118): a block takes and
returns the pair (residual stream ``h``, pending branch output ``d`` or None)."""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..config.base import ScheduleEntry
from .registry import register_part
from .runtime import StepContext


@register_part("block", "pre_norm")
class PreNormBlock:
    def __init__(self, mixer, ffn, norm_mixer, norm_ffn):
        self.mixer, self.ffn, self.norm_mixer, self.norm_ffn = mixer, ffn, norm_mixer, norm_ffn

    def forward(self, h: torch.Tensor, d: Optional[torch.Tensor], ctx: StepContext,
                entry: ScheduleEntry) -> Tuple[torch.Tensor, torch.Tensor]:
        n = self.norm_mixer.forward(h) if d is None else self.norm_mixer.add_forward(h, d)
        a = self.mixer.forward(n, ctx, entry)
        n = self.norm_ffn.add_forward(h, a)
        return h, self.ffn.forward(n, ctx)
