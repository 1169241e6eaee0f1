from .engine_config import EngineConfig
from .model_config import read_config_json
from .registry import (
    Architecture,
    architecture_for,
    load_model_config,
    register_architecture,
    registered_architectures,
    unregister_architecture,
)

__all__ = [
    "Architecture",
    "EngineConfig",
    "architecture_for",
    "load_model_config",
    "read_config_json",
    "register_architecture",
    "registered_architectures",
    "unregister_architecture",
]
