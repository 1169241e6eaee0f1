"""Data that describes a model: which parts, with which sizes, in which order.

A model is not a class hierarchy here.  An architecture's builder turns its typed
configuration into a ``ModelSpec``: one ``LayerSpec`` per set of layer weights
(each naming its mixer, feed-forward, norms and their arrangement, with all sizes
and constants as parameters) and an ``order`` list that says which layers run, in
which sequence, and which cache stream each run reads and writes.  The order may
name a layer twice, and a run may read the cache stream another run wrote.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """One part: ``kind`` selects the class in the part registry, ``params`` are its sizes."""

    kind: str
    params: dict = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part expects in the checkpoint (src/model_config.cpp:78-97).

    ``init`` names the rule of the random-weights mode: "matrix" draws N(0, std),
    "norm" draws 1 + N(0, std), "zeros" and "ones" are constant.
    ``optional`` tensors may be absent (a tied output head).
    """

    name: str
    shape: tuple[int, ...]
    init: str = "matrix"
    std: float = 0.02
    optional: bool = False
    integer: bool = False


@dataclass(frozen=True)
class LayerSpec:
    """One set of layer weights: tensor-name prefix and the block that arranges the parts."""

    prefix: str
    block: PartSpec


@dataclass(frozen=True)
class OrderEntry:
    """One run of a layer.

    layer         index into ``ModelSpec.layers`` (the weights that run).
    cache         id of the cache stream this run uses; runs with the same id
                  share one cache, so a run may read what another run wrote.
    writes_cache  False for a run that only reads a stream another run filled.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    order: tuple[OrderEntry, ...]
    final_norm: PartSpec
    head: PartSpec

    def validate(self) -> None:
        from ..errors import ConfigError

        writers: dict[int, int] = {}
        for index, entry in enumerate(self.order):
            if not 0 <= entry.layer < len(self.layers):
                raise ConfigError(f"order entry {index} names layer {entry.layer}, which does not exist")
            if entry.writes_cache:
                if entry.cache in writers:
                    raise ConfigError(
                        f"order entries {writers[entry.cache]} and {index} both write cache stream {entry.cache}"
                    )
                writers[entry.cache] = index
        for index, entry in enumerate(self.order):
            if not entry.writes_cache:
                if entry.cache not in writers or writers[entry.cache] > index:
                    raise ConfigError(
                        f"order entry {index} reads cache stream {entry.cache} before any run wrote it"
                    )
