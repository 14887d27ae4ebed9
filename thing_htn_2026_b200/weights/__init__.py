from .loader import (GAIN, MATRIX, TABLE, TensorSpec, UndeclaredTensorsWarning, WeightError, held_dtype,
                     load_tensors, merge_specs)
from .random_init import (INITIALIZERS, random_tensors_cpu, random_tensors_on_device, register_initializer,
                          write_random_model)
from .safetensors_io import Checkpoint, SafetensorsError, SafetensorsFile, write_safetensors

__all__ = [
    "GAIN", "MATRIX", "TABLE", "TensorSpec", "UndeclaredTensorsWarning", "WeightError", "held_dtype", "load_tensors", "merge_specs",
    "INITIALIZERS", "register_initializer", "random_tensors_cpu", "random_tensors_on_device", "write_random_model",
    "Checkpoint", "SafetensorsError", "SafetensorsFile", "write_safetensors",
]
