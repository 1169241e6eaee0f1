from . import attention, block, ends, mlp, norm, position  # noqa: F401  (registers the built-in parts)
from .base import (
    Block,
    CacheNeed,
    FeedForward,
    LayerCache,
    Mixer,
    Norm,
    Part,
    PositionEncoding,
    Runtime,
    Workspace,
    build_part,
    norm_then_part,
    part_class,
    register_part,
    unregister_part,
)
from .spec import LayerSpec, ModelSpec, OrderEntry, PartSpec, TensorSpec

__all__ = [
    "Block", "CacheNeed", "FeedForward", "LayerCache", "LayerSpec", "Mixer", "ModelSpec", "Norm", "OrderEntry",
    "Part", "PartSpec", "PositionEncoding", "Runtime", "TensorSpec", "Workspace", "build_part", "norm_then_part", "part_class",
    "register_part", "unregister_part",
]
