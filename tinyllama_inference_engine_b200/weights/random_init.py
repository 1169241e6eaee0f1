"""Random-weights mode: write a model folder from a configuration and a seed.

The reference has no such mode (its microbenchmark fills buffers with a sine
pattern, benchmarks/kernel_benchmarks.cu:80-92).  Matrices are N(0, std) and norm
weights 1 + N(0, std), drawn in 32-bit from ONE seeded generator consumed in the
order of the expected-tensor list, then rounded to the storage dtype, so that a
plain implementation reading the folder sees exactly the values the engine sees.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Iterable

import torch

from ..errors import ConfigError
from ..parts.spec import TensorSpec
from .safetensors_io import write_safetensors

_STORAGE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def random_tensors(expected: Iterable[TensorSpec], seed: int, dtype: torch.dtype = torch.bfloat16) -> dict[str, torch.Tensor]:
    generator = torch.Generator(device="cpu")
    generator.manual_seed(int(seed))
    tensors: dict[str, torch.Tensor] = {}
    for spec in expected:
        if spec.optional:
            continue
        if spec.init == "matrix":
            value = torch.randn(spec.shape, generator=generator, dtype=torch.float32) * spec.std
        elif spec.init == "norm":
            value = 1.0 + torch.randn(spec.shape, generator=generator, dtype=torch.float32) * spec.std
        elif spec.init == "zeros":
            value = torch.zeros(spec.shape, dtype=torch.float32)
        elif spec.init == "ones":
            value = torch.ones(spec.shape, dtype=torch.float32)
        else:
            raise ConfigError(f"unknown init rule {spec.init!r} for {spec.name}")
        tensors[spec.name] = value.to(torch.int32) if spec.integer else value.to(dtype)
    return tensors


def write_random_model(folder: str | Path, config: Any, seed: int, storage_dtype: str | None = None) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (any registered architecture).

    ``config`` is a typed configuration or the dictionary of a config.json, which the registry turns into one."""
    from ..config.registry import architecture_for
    from ..models.model import expected_tensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    if isinstance(config, dict):
        config = architecture_for(config).config_class.from_dict(config)
    data = config.to_dict()
    architecture = architecture_for(data)
    spec = architecture.build_spec(config)
    name = storage_dtype or data.get("torch_dtype") or "bfloat16"
    if name not in _STORAGE:
        raise ConfigError(f"cannot write random weights as {name!r}")
    tensors = random_tensors(expected_tensors(spec), seed, _STORAGE[name])
    (folder / "config.json").write_text(json.dumps(data, indent=2) + "\n")
    write_safetensors(folder / "model.safetensors", tensors, metadata={"format": "pt", "seed": seed})
    return folder
