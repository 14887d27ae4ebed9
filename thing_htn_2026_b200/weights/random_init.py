"""Random weights from a configuration and a seed.

Distributions: matrices and the embedding table N(0, ``matrix_std``); norm gains
1 + N(0, ``gain_std``).  (The reference draws random weights only in kernel
self-tests, N(0, 0.02) with gains around 1: engine/kernels/gemm_fused.py:209-219,
engine/kernels/rmsnorm.py:258-260.)  Every tensor has a generator of its own, seeded
from (seed, position of the tensor in the model's declaration order), so a tensor's
values do not depend on the others.

:func:`write_random_model` writes a model folder (config.json, model.safetensors);
:func:`random_tensors_on_device` fills a large model directly on the GPU.
"""

from __future__ import annotations

import json
import os
from typing import Callable, Dict, Iterable

import torch

from ..config.base import ModelConfig
from .loader import GAIN, MATRIX, TABLE, TensorSpec, held_dtype, merge_specs
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, index: int) -> int:
    return (int(seed) * 1_000_003 + index * 7919 + 12345) % (2 ** 63 - 1)


def _normal(t, generator, matrix_std, gain_std):
    return t.normal_(0.0, matrix_std, generator=generator)


def _one_plus_normal(t, generator, matrix_std, gain_std):
    return t.normal_(0.0, gain_std, generator=generator).add_(1.0)


def _zeros(t, generator, matrix_std, gain_std):
    return t.zero_()


# How a tensor is drawn, by the name in ``TensorSpec.init``.  ``fill(t, generator, matrix_std,
# gain_std)`` fills ``t`` (float32 on the CPU, the held dtype on a device) in place.
INITIALIZERS: Dict[str, Callable] = {"normal": _normal, "one_plus_normal": _one_plus_normal, "zeros": _zeros}
# The rule of a spec that names none, by its role.
ROLE_INIT = {MATRIX: "normal", GAIN: "one_plus_normal", TABLE: "zeros"}


def register_initializer(name: str, fill: Callable) -> None:
    """A new drawing rule (a gain stored as ``w`` of ``1 + w``, a bias, ...) for specs that
    name it in ``TensorSpec.init``."""
    if name in INITIALIZERS and INITIALIZERS[name] is not fill:
        raise ValueError(f"initializer '{name}' is already registered")
    INITIALIZERS[name] = fill


def _draw(spec: TensorSpec, generator: torch.Generator, device, matrix_std: float, gain_std: float,
          dtype: torch.dtype) -> torch.Tensor:
    rule = spec.init or ROLE_INIT.get(spec.role)
    if rule not in INITIALIZERS:
        raise KeyError(f"{spec.name}: no initializer named '{rule}' (role '{spec.role}'); known: "
                       + ", ".join(sorted(INITIALIZERS)))
    if spec.role == TABLE:
        return INITIALIZERS[rule](torch.zeros(spec.shape, dtype=torch.int32, device=device), generator,
                                  matrix_std, gain_std)
    t = torch.empty(spec.shape, dtype=torch.float32 if device == "cpu" else dtype, device=device)
    return INITIALIZERS[rule](t, generator, matrix_std, gain_std).to(dtype)


def specs_of(config: ModelConfig) -> Dict[str, TensorSpec]:
    from ..models.decoder import tensor_specs_of_plan
    return merge_specs(tensor_specs_of_plan(config.plan()))


def random_tensors_cpu(config: ModelConfig, seed: int, dtype: torch.dtype = torch.float32,
                       matrix_std: float = 0.02, gain_std: float = 0.1) -> Dict[str, torch.Tensor]:
    out = {}
    for index, spec in enumerate(specs_of(config).values()):
        g = torch.Generator(device="cpu").manual_seed(_tensor_seed(seed, index))
        out[spec.name] = _draw(spec, g, "cpu", matrix_std, gain_std, dtype)
    return out


def write_random_model(model_dir: str, config: ModelConfig, seed: int, dtype: torch.dtype = torch.float32,
                       matrix_std: float = 0.02, gain_std: float = 0.1, device="cpu") -> str:
    """Write config.json and model.safetensors; returns the folder.  ``device``: where the
    values are drawn (a GPU draws a large model in seconds; its generator gives other values
    than the CPU's for the same seed)."""
    os.makedirs(model_dir, exist_ok=True)
    data = config.to_dict()
    data["torch_dtype"] = {torch.float32: "float32", torch.bfloat16: "bfloat16",
                           torch.float16: "float16"}[dtype]
    with open(os.path.join(model_dir, "config.json"), "w") as handle:
        json.dump(data, handle, indent=1)
    if str(device) == "cpu":
        tensors = random_tensors_cpu(config, seed, dtype, matrix_std, gain_std)
    else:
        from ..models.decoder import tensor_specs_of_plan
        drawn = random_tensors_on_device(tensor_specs_of_plan(config.plan()), seed, dtype, torch.device(device),
                                         matrix_std, gain_std)
        tensors = {name: t.to(dtype).cpu() for name, t in drawn.items()}
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return model_dir


def random_tensors_on_device(specs: Iterable[TensorSpec], seed: int, compute_dtype: torch.dtype,
                             device: torch.device, matrix_std: float = 0.02,
                             gain_std: float = 0.02) -> Dict[str, torch.Tensor]:
    """Same distributions drawn by the device generator, tensor by tensor, in the held dtype."""
    out = {}
    for index, spec in enumerate(merge_specs(specs).values()):
        g = torch.Generator(device=device).manual_seed(_tensor_seed(seed, index))
        dtype = held_dtype(compute_dtype, spec.role, compute_dtype)
        out[spec.name] = _draw(spec, g, device, matrix_std, gain_std, dtype)
    return out
