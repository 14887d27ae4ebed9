from .generation import Completion, GenerationLoop, Request, form_batches, tokens_needed

__all__ = ["Completion", "GenerationLoop", "Request", "form_batches", "tokens_needed", "Engine"]


def __getattr__(name):
    if name == "Engine":
        from .engine import Engine
        return Engine
    raise AttributeError(name)
