"""Configurations by name: config.json files kept as data beside the package (the two
tiny test sizes and the layer sizes of Qwen3-4B, -8B and -14B), for the random-weights
mode of the command line and for measurements.  No size lives in code: a preset is a
config.json like any other and goes through the same typed reader."""

from __future__ import annotations

import json
import os
from typing import List

from .base import ConfigError

_FOLDER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "presets")


def named_configs() -> List[str]:
    return sorted(name[:-5] for name in os.listdir(_FOLDER) if name.endswith(".json"))


def named_config_json(name: str) -> dict:
    path = os.path.join(_FOLDER, f"{name.lower()}.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no configuration named '{name}'; known: {', '.join(named_configs())}")
    with open(path) as handle:
        return json.load(handle)
