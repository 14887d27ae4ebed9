"""Weights by tensor name: what the model expects, checked against what a folder holds.

Each part of a model declares the tensors it needs as :class:`TensorSpec` (full
checkpoint name, shape, role).  :func:`load_tensors` reads exactly those.  A missing
tensor or a wrong shape raises ONE :class:`WeightError` that lists every missing tensor,
every wrong shape and every tensor of the file that no part declared.  Tensors that no
part declared are, by themselves, no error: they are listed once in a warning
(:class:`UndeclaredTensorsWarning`) and left unread, as the reference's library loader
accepts whatever else a file holds (engine/engine.py:188-207); ``strict=True`` makes them
fatal.  Names matching the plan's ``ignored_tensors`` patterns are passed over in silence.
A spec may name ``copies``: other names under which some writers store the same tensor
again (a tied head stored beside the embedding, which the reference recognises by
pointer equality after loading, engine/engine.py:225-226).  A stored copy is accepted,
compared with the tensor it duplicates, and reported in the warning if it differs.

Precision rule.  With compute dtype bfloat16: matrices (operands of the tensor-core
products and the embedding table) are held in bfloat16; any other floating tensor that
the file stores in 32 bits stays in 32 bits, one stored in 16 bits becomes bfloat16.
With compute dtype float32 every floating tensor is float32.  Integer tensors become
int32.

Tensor names are the ones the reference reaches through its loader's module tree
(engine/engine.py:208-227; table OPTIMIZATION_GUIDE.md:116-131).
"""

from __future__ import annotations

import fnmatch
import warnings
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .safetensors_io import Checkpoint

MATRIX = "matrix"   # [out, in] operand of a matrix product, or an embedding table
GAIN = "gain"       # multiplicative vector of a norm
TABLE = "table"     # integer table


@dataclass(frozen=True)
class TensorSpec:
    """``role`` decides the precision a tensor is held in; ``init`` names the rule that draws
    it in the random-weights mode (None: the role's default, see weights/random_init.py);
    ``copies`` are other checkpoint names that may store the same tensor once more."""

    name: str
    shape: Tuple[int, ...]
    role: str = MATRIX
    init: Optional[str] = None
    copies: Tuple[str, ...] = ()


class UndeclaredTensorsWarning(UserWarning):
    """The checkpoint holds tensors that no part of the model reads."""


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
        elif spec.copies and set(spec.copies) - set(seen.copies):
            merged[spec.name] = TensorSpec(seen.name, seen.shape, seen.role, seen.init,
                                           tuple(dict.fromkeys(seen.copies + spec.copies)))
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


def check_names(where: str, specs: Dict[str, TensorSpec], found: Dict[str, Tuple[int, ...]],
                ignored: Sequence[str] = (), strict: bool = False) -> List[str]:
    """Raises the one :class:`WeightError`, or returns the undeclared names (copies and
    ignored patterns left out) for the caller to warn about."""
    copies = {c: s for s in specs.values() for c in s.copies}
    missing = [n for n in specs if n not in found]
    unexpected = [n for n in found if n not in specs and n not in copies
                  and not any(fnmatch.fnmatchcase(n, pattern) for pattern in ignored)]
    wrong = [(n, tuple(found[n]), tuple(s.shape)) for n, s in specs.items()
             if n in found and tuple(found[n]) != tuple(s.shape)]
    wrong += [(c, tuple(found[c]), tuple(s.shape)) for c, s in copies.items()
              if c in found and tuple(found[c]) != tuple(s.shape)]
    if missing or wrong or (strict and unexpected):
        raise WeightError(where, missing, unexpected, wrong)
    return unexpected


def load_tensors(model_dir: str, specs: Iterable[TensorSpec], compute_dtype: torch.dtype,
                 device: torch.device, ignored: Sequence[str] = (), strict: bool = False) -> Dict[str, torch.Tensor]:
    merged = merge_specs(specs)
    checkpoint = Checkpoint(model_dir)
    undeclared = check_names(model_dir, merged, {n: e.shape for n, e in checkpoint.entries.items()}, ignored, strict)
    notes: List[str] = []
    if undeclared:
        notes.append(f"{len(undeclared)} tensors that no part of the model reads were left unread: "
                     + ", ".join(undeclared))
    out: Dict[str, torch.Tensor] = {}
    for name, spec in merged.items():
        tensor = checkpoint.read(name)
        for copy in spec.copies:
            if copy in checkpoint.entries and not torch.equal(checkpoint.read(copy), tensor):
                notes.append(f"{copy} is stored beside {name}, which the model uses in its place, "
                             f"and differs from it")
        out[name] = tensor.to(device=device, dtype=held_dtype(tensor.dtype, spec.role, compute_dtype)).contiguous()
    if notes:
        warnings.warn(f"{model_dir}: " + "; ".join(notes), UndeclaredTensorsWarning, stacklevel=2)
    return out
