"""Weights by tensor name: what the model expects, checked against what a folder holds.

Each part of a model declares the tensors it needs as :class:`TensorSpec` (full
checkpoint name, shape, role).  :func:`load_tensors` reads exactly those, and raises
ONE :class:`WeightError` that lists every missing tensor, every unexpected tensor and
every wrong shape.

Precision rule.  With compute dtype bfloat16: matrices (operands of the tensor-core
products and the embedding table) are held in bfloat16; any other floating tensor that
the file stores in 32 bits stays in 32 bits, one stored in 16 bits becomes bfloat16.
With compute dtype float32 every floating tensor is float32.  Integer tensors become
int32.

Tensor names are the ones the reference reaches through its loader's module tree
(engine/engine.py:208-227; table OPTIMIZATION_GUIDE.md:116-131).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Sequence, Tuple

import torch

from .safetensors_io import Checkpoint

MATRIX = "matrix"   # [out, in] operand of a matrix product, or an embedding table
GAIN = "gain"       # multiplicative vector of a norm
TABLE = "table"     # integer table


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: Tuple[int, ...]
    role: str = MATRIX


class WeightError(ValueError):
    """The checkpoint does not match the model; lists all differences at once."""

    def __init__(self, where: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 conflicts: Sequence[str] = ()):
        self.missing, self.unexpected, self.wrong = list(missing), list(unexpected), list(wrong)
        self.conflicts = list(conflicts)
        lines = [f"{where}: checkpoint does not match the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong:
            lines.append(f"  wrong shapes ({len(self.wrong)}): " + "; ".join(
                f"{n}: file {list(got)}, model {list(want)}" for n, got, want in self.wrong))
        if self.conflicts:
            lines.append("  conflicting declarations: " + "; ".join(self.conflicts))
        super().__init__("\n".join(lines))


def merge_specs(specs: Iterable[TensorSpec]) -> Dict[str, TensorSpec]:
    """Collapse specs that name the same tensor (a tied head names the embedding)."""
    merged: Dict[str, TensorSpec] = {}
    conflicts: List[str] = []
    for spec in specs:
        seen = merged.get(spec.name)
        if seen is None:
            merged[spec.name] = spec
        elif seen.shape != spec.shape:
            conflicts.append(f"{spec.name}: {list(seen.shape)} vs {list(spec.shape)}")
    if conflicts:
        raise WeightError("model", [], [], [], conflicts)
    return merged


def held_dtype(stored: torch.dtype, role: str, compute_dtype: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if compute_dtype == torch.float32:
        return torch.float32
    if role == MATRIX:
        return compute_dtype
    return torch.float32 if stored in (torch.float32, torch.float64) else compute_dtype


def check_names(where: str, specs: Dict[str, TensorSpec], found: Dict[str, Tuple[int, ...]]) -> None:
    missing = [n for n in specs if n not in found]
    unexpected = [n for n in found if n not in specs]
    wrong = [(n, tuple(found[n]), tuple(s.shape)) for n, s in specs.items()
             if n in found and tuple(found[n]) != tuple(s.shape)]
    if missing or unexpected or wrong:
        raise WeightError(where, missing, unexpected, wrong)


def load_tensors(model_dir: str, specs: Iterable[TensorSpec], compute_dtype: torch.dtype,
                 device: torch.device) -> Dict[str, torch.Tensor]:
    merged = merge_specs(specs)
    checkpoint = Checkpoint(model_dir)
    check_names(model_dir, merged, {n: e.shape for n, e in checkpoint.entries.items()})
    out: Dict[str, torch.Tensor] = {}
    for name, spec in merged.items():
        tensor = checkpoint.read(name)
        out[name] = tensor.to(device=device, dtype=held_dtype(tensor.dtype, spec.role, compute_dtype)).contiguous()
    return out
