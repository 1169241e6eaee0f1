"""Options of the engine itself: nothing here comes from the checkpoint."""
from __future__ import annotations

from dataclasses import dataclass

from ..errors import ConfigError

DTYPES = ("bfloat16", "float32")


@dataclass
class EngineConfig:
    """How the model is run.

    dtype             "bfloat16": bf16 weights, activations and cache with 32-bit
                      softmax, norms, rotation and residual; "float32": everything
                      in true 32-bit.
    page_size         tokens per cache page (a multiple of 16).
    max_cache_tokens  capacity of every cache group's page pool, in tokens.
    max_requests      live requests (state slots and block-table rows).
    max_batch_tokens  token budget of one step (the scheduler cuts prompts to it).
    weights_sha256    if given, the SHA-256 the model folder's weights must have (weights/integrity.py); loading a folder
                      with another digest fails with ``checksum_mismatch``.
    """

    dtype: str = "bfloat16"
    page_size: int = 64
    max_cache_tokens: int = 8192
    max_requests: int = 64
    max_batch_tokens: int = 2048
    device: str = "cuda:0"
    use_cuda_graphs: bool = True
    poison_freed_pages: bool = False
    weights_sha256: str | None = None

    def __post_init__(self) -> None:
        if self.dtype in ("bf16", "fp32"):
            self.dtype = {"bf16": "bfloat16", "fp32": "float32"}[self.dtype]
        if self.dtype not in DTYPES:
            raise ConfigError(f"dtype must be one of {DTYPES}, got {self.dtype!r}")
        if self.page_size < 16 or self.page_size % 16 != 0:
            raise ConfigError(f"page_size must be a positive multiple of 16, got {self.page_size}")
        if self.max_cache_tokens < self.page_size:
            raise ConfigError("max_cache_tokens must hold at least one page")
        if self.max_requests < 1 or self.max_batch_tokens < 1:
            raise ConfigError("max_requests and max_batch_tokens must be positive")

    @property
    def num_pages(self) -> int:
        return self.max_cache_tokens // self.page_size
