"""Architecture-neutral description of a decoder: parts, layers and the order they run in.

A configuration class reads one architecture's ``config.json`` keys and turns them
into a :class:`ModelPlan`.  The plan is plain data: every size and constant the
kernels need is a parameter of some :class:`PartSpec`; nothing below the
configuration layer knows which architecture it serves.

The reference reads the same keys into untyped attributes
(engine/engine.py:128-141); here they are typed, validated and carried as data.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any, Mapping, Tuple


class ConfigError(ValueError):
    """A config.json that this library cannot run, with the offending key named."""


def _freeze(value: Any) -> Any:
    if isinstance(value, PartSpec):
        return value
    if isinstance(value, dict):
        return MappingProxyType({k: _freeze(v) for k, v in value.items()})
    if isinstance(value, list):
        return tuple(_freeze(v) for v in value)
    return value


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: ``kind`` selects the class in the part registry,
    ``params`` are its sizes and constants, ``tensors`` maps the part's own
    parameter names to full tensor names in the checkpoint."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    tensors: Mapping[str, str] = field(default_factory=dict)

    def __post_init__(self):
        object.__setattr__(self, "params", _freeze(dict(self.params)))
        object.__setattr__(self, "tensors", _freeze(dict(self.tensors)))

    def key(self) -> str:
        """Stable text form, used to share identical parts (e.g. one RoPE table)."""
        def enc(v):
            if isinstance(v, PartSpec):
                return {"kind": v.kind, "params": enc(v.params), "tensors": enc(v.tensors)}
            if isinstance(v, Mapping):
                return {k: enc(x) for k, x in sorted(v.items())}
            if isinstance(v, tuple):
                return [enc(x) for x in v]
            return v
        return json.dumps(enc(self), sort_keys=True)


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: a part of the ``block`` family.  The block owns its sub-parts:
    its ``params`` hold their specs (for the ``pre_norm`` arrangement: ``mixer``, ``ffn``,
    ``norm_mixer``, ``norm_ffn``), so an arrangement with other members (a third norm, no
    feed-forward, two mixers side by side) is a new block class and nothing else."""

    block: PartSpec

    @classmethod
    def of(cls, kind: str, **parts: Any) -> "LayerSpec":
        """``LayerSpec.of("pre_norm", mixer=..., ffn=..., norm_mixer=..., norm_ffn=...)``: a
        block of that kind whose parameters are the given sub-part specs (and constants)."""
        return cls(PartSpec(kind, parts))

    def part(self, name: str) -> PartSpec:
        """A sub-part's spec by its name among the block's parameters."""
        value = self.block.params.get(name)
        if not isinstance(value, PartSpec):
            raise KeyError(f"block '{self.block.kind}' has no part named '{name}'")
        return value


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.

    ``layer`` indexes ``ModelPlan.layers`` (a layer may be named more than once:
    its weights are then shared).  ``cache`` is the id of the cache entry the
    mixer works on; two schedule entries with the same ``cache`` share it, and
    only the entry with ``writes_cache`` appends to it (the other one reads what
    the first wrote).
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelPlan:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    max_positions: int
    # Name patterns (fnmatch) of checkpoint tensors that no part reads and the loader passes
    # over in silence: buffers that some writers store beside the weights.
    ignored_tensors: Tuple[str, ...] = ()

    def __post_init__(self):
        n_layers = len(self.layers)
        writers = {}
        for i, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < n_layers:
                raise ConfigError(f"schedule[{i}] names layer {entry.layer}, plan has {n_layers} layers")
            if entry.writes_cache:
                if entry.cache in writers:
                    raise ConfigError(
                        f"schedule[{i}] and schedule[{writers[entry.cache]}] both write cache {entry.cache}")
                writers[entry.cache] = i
        for i, entry in enumerate(self.schedule):
            if not entry.writes_cache:
                if entry.cache not in writers or writers[entry.cache] > i:
                    raise ConfigError(
                        f"schedule[{i}] reads cache {entry.cache} before any entry has written it")

    @property
    def n_cache_entries(self) -> int:
        return 1 + max((e.cache for e in self.schedule), default=-1)


class ModelConfig:
    """Base of the typed configurations.  Subclasses are dataclasses whose fields
    are config.json keys; they implement :meth:`from_dict`, :meth:`to_dict` and
    :meth:`plan`."""

    architecture: str = ""

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict:
        raise NotImplementedError

    def plan(self) -> ModelPlan:
        raise NotImplementedError


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path) as handle:
            data = json.load(handle)
    except FileNotFoundError:
        raise ConfigError(f"{path}: not found (a model folder holds config.json and model.safetensors)") from None
    except json.JSONDecodeError as error:
        raise ConfigError(f"{path}: not valid JSON ({error})") from None
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return data


def require(data: Mapping[str, Any], key: str, kind, *, positive: bool = True):
    """Fetch a required key of a given type; name the key in the error."""
    if key not in data or data[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    value = data[key]
    if kind is float and isinstance(value, int) and not isinstance(value, bool):
        value = float(value)
    if kind is int and isinstance(value, bool) or not isinstance(value, kind):
        raise ConfigError(f"config.json: '{key}' must be {kind.__name__}, got {value!r}")
    if positive and value <= 0:
        raise ConfigError(f"config.json: '{key}' must be positive, got {value!r}")
    return value
