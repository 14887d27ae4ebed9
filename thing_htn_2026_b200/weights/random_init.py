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
from typing import Dict, Iterable

import torch

from ..config.base import ModelConfig
from .loader import GAIN, MATRIX, TABLE, TensorSpec, held_dtype, merge_specs
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, index: int) -> int:
    return (int(seed) * 1_000_003 + index * 7919 + 12345) % (2 ** 63 - 1)


def _draw(spec: TensorSpec, generator: torch.Generator, device, matrix_std: float, gain_std: float,
          dtype: torch.dtype) -> torch.Tensor:
    if spec.role == TABLE:
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    t = torch.empty(spec.shape, dtype=torch.float32 if device == "cpu" else dtype, device=device)
    if spec.role == GAIN:
        t.normal_(0.0, gain_std, generator=generator).add_(1.0)
    else:
        t.normal_(0.0, matrix_std, generator=generator)
    return t.to(dtype)


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
                       matrix_std: float = 0.02, gain_std: float = 0.1) -> str:
    """Write config.json and model.safetensors; returns the folder."""
    os.makedirs(model_dir, exist_ok=True)
    data = config.to_dict()
    data["torch_dtype"] = {torch.float32: "float32", torch.bfloat16: "bfloat16",
                           torch.float16: "float16"}[dtype]
    with open(os.path.join(model_dir, "config.json"), "w") as handle:
        json.dump(data, handle, indent=1)
    tensors = random_tensors_cpu(config, seed, dtype, matrix_std, gain_std)
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
