"""Qwen3 dense generation for one NVIDIA B200 (sm_100a): configuration, weights, parts,
cache, step function, generation loop, sampling and the CUDA kernels under them."""

__version__ = "0.1.0"


def __getattr__(name):
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    raise AttributeError(name)
