from .loader import GAIN, MATRIX, TABLE, TensorSpec, WeightError, held_dtype, load_tensors, merge_specs
from .random_init import random_tensors_cpu, random_tensors_on_device, write_random_model
from .safetensors_io import Checkpoint, SafetensorsError, SafetensorsFile, write_safetensors

__all__ = [
    "GAIN", "MATRIX", "TABLE", "TensorSpec", "WeightError", "held_dtype", "load_tensors", "merge_specs",
    "random_tensors_cpu", "random_tensors_on_device", "write_random_model",
    "Checkpoint", "SafetensorsError", "SafetensorsFile", "write_safetensors",
]
