"""Grouped-query attention over the cache: the token mixer of this architecture.

One product gives q, k and v (weights concatenated ``[q; k; v]`` as the reference does,
engine/engine.py:214-216); one kernel normalises q and k per head, rotates them and writes
K and V to the cache (engine/kernels/torch_ref.py:107-162); attention then reads the
cache, which already holds the step's own keys (engine/kernels/torch_ref.py:168-227);
one product projects back (engine/engine.py:1114).

Parameters (all from the PartSpec): ``hidden_size, n_heads, n_kv_heads, head_dim, scale``,
``window`` (None: all keys; W: the last W keys), ``qk_norm_eps`` (None: no head norm) and
``position`` (a position PartSpec or None).  A schedule entry with ``writes_cache=False``
makes the mixer read the cache another entry wrote: it computes only its queries.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..cache.sequence_cache import CacheNeed, KVSpec
from ..config.base import PartSpec, ScheduleEntry
from ..weights.loader import GAIN, MATRIX, TensorSpec
from .registry import part_class, register_part
from .runtime import HostBatch, Runtime, StepContext


@register_part("mixer", "attention")
class Attention:
    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        p = spec.params
        hidden, n_q, n_kv, d = int(p["hidden_size"]), int(p["n_heads"]), int(p["n_kv_heads"]), int(p["head_dim"])
        specs = [TensorSpec(spec.tensors["q_proj"], (n_q * d, hidden), MATRIX),
                 TensorSpec(spec.tensors["k_proj"], (n_kv * d, hidden), MATRIX),
                 TensorSpec(spec.tensors["v_proj"], (n_kv * d, hidden), MATRIX),
                 TensorSpec(spec.tensors["o_proj"], (hidden, n_q * d), MATRIX)]
        if p.get("qk_norm_eps") is not None:
            specs += [TensorSpec(spec.tensors["q_norm"], (d,), GAIN), TensorSpec(spec.tensors["k_norm"], (d,), GAIN)]
        return specs

    def __init__(self, spec: PartSpec, runtime: Runtime):
        p = spec.params
        self.n_q, self.n_kv, self.head_dim = int(p["n_heads"]), int(p["n_kv_heads"]), int(p["head_dim"])
        if self.n_q % self.n_kv:
            raise ValueError(f"attention: {self.n_q} heads are not a multiple of {self.n_kv} kv heads")
        self.scale = float(p["scale"])
        self.window: Optional[int] = None if p.get("window") is None else int(p["window"])
        self.eps = None if p.get("qk_norm_eps") is None else float(p["qk_norm_eps"])
        self.w_qkv = torch.cat([runtime.tensor(spec, "q_proj"), runtime.tensor(spec, "k_proj"),
                                runtime.tensor(spec, "v_proj")], dim=0).contiguous()
        self.w_o = runtime.tensor(spec, "o_proj")
        self.q_gain = runtime.tensor(spec, "q_norm") if self.eps is not None else None
        self.k_gain = runtime.tensor(spec, "k_norm") if self.eps is not None else None
        self.dtype = runtime.dtype
        self.position = None
        position_spec = p.get("position")
        if position_spec is not None:
            key = "position:" + position_spec.key()
            if key not in runtime.shared:
                runtime.shared[key] = part_class("position", position_spec.kind)(position_spec, runtime)
            self.position = runtime.shared[key]

    def cache_need(self) -> CacheNeed:
        return KVSpec(self.n_kv, self.head_dim, self.window)

    def _tile(self, page_size: int) -> int:
        return ops.prompt_attention_tile(self.dtype, self.head_dim, page_size, self.n_q, self.n_kv)

    def step_inputs(self, batch: HostBatch, out: Dict[str, List[int]]) -> None:
        """The prompt attention kernels work on tiles of consecutive rows of one sequence; the
        host knows every length, so it lists them (every attention of a model that wants
        tiles of one size shares one list)."""
        size = self._tile(batch.page_size) if batch.max_count > 1 else 0
        if size and f"row_tiles/{size}/row0" not in out:
            out[f"row_tiles/{size}/row0"], out[f"row_tiles/{size}/rows"] = ops.row_tiles_of(
                batch.counts, batch.held, size)

    def forward(self, x: torch.Tensor, ctx: StepContext, entry: ScheduleEntry) -> torch.Tensor:
        kv = ctx.cache.kv_view(entry.cache)
        tiles = None
        if ctx.rows.max_q_len > 1:
            size = self._tile(kv.page_size)
            row0 = ctx.inputs.get(f"row_tiles/{size}/row0") if size else None
            if row0 is not None:
                tiles = ops.RowTiles(row0, ctx.inputs[f"row_tiles/{size}/rows"], row0.shape[0], size)
        qkv = ops.linear(x, self.w_qkv, err=ctx.err)
        a = ops.qkv_attention(qkv, self.q_gain, self.k_gain, self.eps if self.eps is not None else 1.0,
                              self.position.tables() if self.position is not None else None,
                              ctx.rows, kv, self.n_q, self.scale, self.window, entry.writes_cache, ctx.err, tiles)
        return ops.linear(a, self.w_o, err=ctx.err)
