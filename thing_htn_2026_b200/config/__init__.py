from .base import (ConfigError, LayerSpec, ModelConfig, ModelPlan, PartSpec, ScheduleEntry,
                   read_config_json)
from .named import named_config_json, named_configs
from .qwen3 import Qwen3Config
from .registry import (architecture_of, config_from_dict, known_architectures, load_config,
                       model_class_for, register_architecture)

__all__ = [
    "ConfigError", "LayerSpec", "ModelConfig", "ModelPlan", "PartSpec", "ScheduleEntry",
    "read_config_json", "Qwen3Config", "named_config_json", "named_configs", "architecture_of", "config_from_dict",
    "known_architectures", "load_config", "model_class_for", "register_architecture",
]
