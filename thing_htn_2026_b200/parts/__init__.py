from . import attention, block, embedding, feedforward, norms, positions  # noqa: F401  (registration)
from .registry import FAMILIES, part_class, register_part, unregister_part
from .block import Block
from .runtime import HostBatch, Runtime, StepContext

__all__ = ["FAMILIES", "part_class", "register_part", "unregister_part", "Block", "HostBatch", "Runtime", "StepContext"]
