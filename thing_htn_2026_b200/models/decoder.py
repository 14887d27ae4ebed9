"""A decoder assembled from a :class:`ModelPlan`: embedding, the scheduled layers, final
norm, head.  Nothing here knows an architecture's name; the plan decides the parts, their
sizes and the order in which layers run (the reference's fixed loop is
engine/engine.py:1101-1121)."""

from __future__ import annotations

from typing import Dict, Iterable, List, Optional

import torch

from .. import ops
from ..cache.sequence_cache import CacheNeed
from ..config.base import ModelConfig, ModelPlan, PartSpec
from ..parts import HostBatch, Runtime, StepContext, part_class
from ..weights.loader import TensorSpec, load_tensors, merge_specs
from ..weights.random_init import random_tensors_on_device


def tensor_specs_of_plan(plan: ModelPlan) -> List[TensorSpec]:
    """Every tensor the plan's parts declare, in declaration order."""
    specs: List[TensorSpec] = list(part_class("embedding", plan.embedding.kind).tensor_specs(plan.embedding))
    for layer in plan.layers:
        specs += part_class("block", layer.block.kind).tensor_specs(layer.block)
    specs += part_class("norm", plan.final_norm.kind).tensor_specs(plan.final_norm)
    specs += part_class("head", plan.head.kind).tensor_specs(plan.head)
    return specs


class DecoderModel:
    def __init__(self, config: ModelConfig, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device):
        self.config = config
        self.plan = plan = config.plan()
        self.dtype = dtype
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ops.KernelError(f"the model runs on CUDA only, got device {self.device}")
        self.runtime = runtime = Runtime(dtype, self.device, tensors)
        self.embedding = part_class("embedding", plan.embedding.kind)(plan.embedding, runtime)
        self.layers = [part_class("block", layer.block.kind)(layer.block, runtime) for layer in plan.layers]
        self.final_norm = part_class("norm", plan.final_norm.kind)(plan.final_norm, runtime)
        self.head = part_class("head", plan.head.kind)(plan.head, runtime)
        self.vocab_size = plan.vocab_size
        runtime.tensors = {}   # parts hold what they need; fused copies replace the originals

    # ------------------------------------------------------------------ construction

    @classmethod
    def from_folder(cls, config: ModelConfig, model_dir: str, dtype: torch.dtype, device) -> "DecoderModel":
        plan = config.plan()
        tensors = load_tensors(model_dir, tensor_specs_of_plan(plan), dtype, torch.device(device),
                               ignored=plan.ignored_tensors)
        return cls(config, tensors, dtype, device)

    @classmethod
    def from_random(cls, config: ModelConfig, seed: int, dtype: torch.dtype, device,
                    matrix_std: float = 0.02, gain_std: float = 0.02) -> "DecoderModel":
        tensors = random_tensors_on_device(tensor_specs_of_plan(config.plan()), seed, dtype, torch.device(device),
                                           matrix_std, gain_std)
        return cls(config, tensors, dtype, device)

    # ------------------------------------------------------------------ cache and positions

    def cache_needs(self) -> List[CacheNeed]:
        """What each cache entry stores: the need of the schedule entry that writes it."""
        needs: List[CacheNeed] = [None] * self.plan.n_cache_entries
        for entry in self.plan.schedule:
            if entry.writes_cache:
                needs[entry.cache] = self.layers[entry.layer].cache_need()
        return needs

    def ensure_positions(self, n_positions: int) -> None:
        for part in self.runtime.shared.values():
            if hasattr(part, "ensure"):
                part.ensure(n_positions)

    def step_inputs(self, batch: HostBatch) -> Dict[str, List[int]]:
        """Integer inputs that parts want computed on the host for this step, by name; the
        step function uploads them with the tokens."""
        out: Dict[str, List[int]] = {}
        for layer in self.layers:
            layer.step_inputs(batch, out)
        return out

    # ------------------------------------------------------------------ forward

    def hidden(self, tokens: torch.Tensor, ctx: StepContext):
        """All scheduled layers over the step's rows; returns the residual stream and the
        last branch output that has not been added yet."""
        h = self.embedding.forward(tokens, ctx.err)
        d: Optional[torch.Tensor] = None
        for entry in self.plan.schedule:
            h, d = self.layers[entry.layer].forward(h, d, ctx, entry)
        return h, d

    def logits(self, h: torch.Tensor, d: Optional[torch.Tensor], rows: Optional[torch.Tensor],
               err: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Final norm and head at the given rows (int32 indices; None: every row): float32.
        ``err``: the step's device error word."""
        if rows is not None:
            h = ops.gather_rows(h, rows)
            d = ops.gather_rows(d, rows) if d is not None else None
        n = self.final_norm.forward(h) if d is None else self.final_norm.add_forward(h, d)
        return self.head.forward(n, err)

    def forward(self, tokens: torch.Tensor, ctx: StepContext, want_rows: Optional[torch.Tensor]) -> torch.Tensor:
        h, d = self.hidden(tokens, ctx)
        return self.logits(h, d, want_rows, ctx.err)
