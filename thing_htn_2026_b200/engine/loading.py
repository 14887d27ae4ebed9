"""From a model folder (or a configuration and a seed) to a model on the device."""

from __future__ import annotations

import torch

from ..config import ModelConfig, load_config, model_class_for

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {name} is not supported (bfloat16 or float32)")
        return name
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype '{name}' is not supported (bfloat16 or float32)") from None


def load_model(model_dir: str, dtype="bfloat16", device="cuda:0"):
    """The model class is chosen by config.json's ``architectures``."""
    config = load_config(model_dir)
    return model_class_for(config).from_folder(config, model_dir, parse_dtype(dtype), device)


def random_model(config: ModelConfig, seed: int = 0, dtype="bfloat16", device="cuda:0", **init):
    return model_class_for(config).from_random(config, seed, parse_dtype(dtype), device, **init)
