"""Structured errors of the engine.

Every failure a caller can provoke carries one of the reference's error codes
(include/tlie/error.hpp:7-20) so that command lines can print the same JSON shape
``{"error": {"code", "message"}}`` as app/reference_cli.cpp:20-25.
"""
from __future__ import annotations

ERROR_CODES = (
    "io",
    "invalid_format",
    "checksum_mismatch",
    "invalid_config",
    "invalid_shape",
    "invalid_dtype",
    "out_of_memory",
    "out_of_bounds",
    "tokenizer",
    "numerical",
    "invalid_argument",
    "cuda",
)


class EngineError(Exception):
    """Base class: ``code`` is one of ERROR_CODES."""

    code = "invalid_argument"

    def __init__(self, message: str, code: str | None = None):
        super().__init__(message)
        if code is not None:
            if code not in ERROR_CODES:
                raise ValueError(f"unknown error code {code!r}")
            self.code = code
        self.message = message

    def to_json(self) -> dict:
        return {"error": {"code": self.code, "message": self.message}}


class ConfigError(EngineError):
    code = "invalid_config"


class WeightError(EngineError):
    code = "invalid_shape"


class FormatError(EngineError):
    code = "invalid_format"


class OutOfPages(EngineError):
    """The page pool of some cache group cannot serve a reservation."""

    code = "out_of_memory"


class BatchError(EngineError):
    code = "out_of_bounds"


class KernelError(EngineError):
    code = "cuda"
