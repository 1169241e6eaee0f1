"""Reading config.json, and the checks every typed configuration needs.

A typed configuration class belongs to its architecture and lives beside that
architecture's builder under ``models/``; this module holds what all of them share:
reading the file (the reference's ``ModelConfig::Load``, src/model_config.cpp:16-24)
and turning JSON values into checked numbers.
"""
from __future__ import annotations

import json
import math
from pathlib import Path
from typing import Any

from ..errors import ConfigError, EngineError


def as_int(name: str, value: Any, minimum: int = 1) -> int:
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"{name} must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError(f"{name} must be >= {minimum}, got {value}")
    return value


def as_float(name: str, value: Any) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"{name} must be a number, got {value!r}")
    value = float(value)
    if not math.isfinite(value) or value <= 0.0:
        raise ConfigError(f"{name} must be finite and positive, got {value}")
    return value


def read_config_json(path: str | Path) -> dict:
    path = Path(path)
    if path.is_dir():
        path = path / "config.json"
    try:
        text = path.read_text()
    except OSError as exc:
        raise EngineError(f"unable to open model config: {path}", code="io") from exc
    try:
        data = json.loads(text)
    except json.JSONDecodeError as exc:
        raise ConfigError(f"invalid model config JSON: {exc}") from exc
    if not isinstance(data, dict):
        raise ConfigError("config.json must hold a JSON object")
    return data
