"""One registry from an architecture's name to what builds its model.

The reference has a single hard-wired class and only checks ``model_type == "llama"``
(src/model_config.cpp:25).  Here config.json's ``architectures[0]`` (or its
``model_type``) selects an ``Architecture``: the typed configuration class and the
function that turns a configuration into a ``ModelSpec``.  Nothing else in the
framework names a model.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from ..errors import ConfigError
from .model_config import read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                      # has from_dict(dict) and to_dict()
    build_spec: Callable[[Any], Any]       # config -> ModelSpec
    model_types: tuple[str, ...] = ()


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(architecture: Architecture, *, replace: bool = False) -> None:
    if architecture.name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture {architecture.name!r} is already registered")
    _ARCHITECTURES[architecture.name] = architecture


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def architecture_for(config: dict) -> Architecture:
    """Choose by ``architectures[0]``, falling back to ``model_type``."""
    names = config.get("architectures") or []
    for name in names:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    model_type = config.get("model_type")
    if not names and model_type is not None:
        for architecture in _ARCHITECTURES.values():
            if model_type in architecture.model_types:
                return architecture
    raise ConfigError(
        f"no registered architecture for architectures={list(names)!r} model_type={model_type!r}; "
        f"known: {', '.join(registered_architectures()) or 'none'}"
    )


def load_model_config(model_dir: str | Path) -> tuple[Architecture, Any]:
    """Read ``model_dir/config.json`` and return (architecture, typed configuration)."""
    data = read_config_json(model_dir)
    architecture = architecture_for(data)
    return architecture, architecture.config_class.from_dict(data)
