from . import llama  # noqa: F401  (registers LlamaForCausalLM)
from .model import DecoderModel, cache_needs, expected_tensors

__all__ = ["DecoderModel", "cache_needs", "expected_tensors"]
