"""One registry from an architecture's name (config.json ``architectures[0]``) to its
typed configuration and model class.

The reference has no registry: it hands the folder to a library loader that dispatches
on the same key (engine/engine.py:185-196).  Here the mapping is explicit, and a new
architecture is one :func:`register_architecture` call.
"""

from __future__ import annotations

from typing import Any, Callable, Dict, Mapping, Tuple, Type

from .base import ConfigError, ModelConfig, read_config_json

_ARCHITECTURES: Dict[str, Tuple[Type[ModelConfig], Callable[[], type]]] = {}


def register_architecture(name: str, config_cls: Type[ModelConfig], model_cls: Callable[[], type]) -> None:
    """``model_cls`` is a zero-argument callable returning the model class, so that
    registering an architecture does not import the device code."""
    if name in _ARCHITECTURES:
        raise ValueError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = (config_cls, model_cls)


def known_architectures() -> Tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def architecture_of(data: Mapping[str, Any]) -> str:
    names = data.get("architectures")
    if not isinstance(names, (list, tuple)) or not names or not isinstance(names[0], str):
        raise ConfigError(
            "config.json: 'architectures' must be a non-empty list of names; known: "
            + ", ".join(known_architectures()))
    if names[0] not in _ARCHITECTURES:
        raise ConfigError(
            f"config.json: architecture '{names[0]}' is not registered; known: "
            + ", ".join(known_architectures()))
    return names[0]


def config_from_dict(data: Mapping[str, Any]) -> ModelConfig:
    return _ARCHITECTURES[architecture_of(data)][0].from_dict(data)


def load_config(model_dir: str) -> ModelConfig:
    return config_from_dict(read_config_json(model_dir))


def model_class_for(config: ModelConfig) -> type:
    if config.architecture not in _ARCHITECTURES:
        raise ConfigError(f"architecture '{config.architecture}' is not registered")
    return _ARCHITECTURES[config.architecture][1]()


def _decoder_model():
    from ..models.decoder import DecoderModel
    return DecoderModel


def _register_builtin() -> None:
    from .qwen3 import Qwen3Config
    register_architecture(Qwen3Config.architecture, Qwen3Config, _decoder_model)


_register_builtin()
