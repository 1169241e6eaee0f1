"""A single-GPU inference engine for the Llama dense decoder, written for NVIDIA B200 (sm_100a).

From a model folder (config.json + model.safetensors) to generated tokens: typed
configuration and an architecture registry, weights by tensor name, layers put
together from parts, a paged cache manager, one step function for mixed batches,
a continuous-batching scheduler, sampling, and hand-written CUDA kernels.
"""
from . import models  # noqa: F401  (registers the built-in architecture and parts)
from .config import EngineConfig
from .errors import EngineError

__all__ = ["EngineConfig", "EngineError", "Engine", "SamplingParams", "generate"]
__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Engine", "SamplingParams", "generate"):
        from .engine import api

        return getattr(api, name)
    raise AttributeError(name)
