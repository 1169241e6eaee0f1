"""WeightStore: tensors of a model folder, by name, checked against what the parts expect.

In the manner of the reference's WeightStore::Load / Get / Validate
(src/weight_store.cpp:118-295): every expected tensor is looked up once, and the
folder is refused with ONE error that lists every missing tensor, every unexpected
tensor and every wrong shape.  Storage rule: a tensor is kept as the file has it
(bfloat16 stays bfloat16, float16 stays float16, 32-bit stays 32-bit), integer tables
become int32.  Parts ask for the dtype they compute in when they are built
(``get(name, dtype)``): the 32-bit engine therefore sees every 16-bit value exactly,
and only the bfloat16 engine rounds a float16 checkpoint (the reference's GPU
checkpoints are float16, scripts/convert_model_fp16.py:23-67) to bfloat16.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Iterable

import torch

from ..errors import EngineError, WeightError
from ..parts.spec import TensorSpec
from .safetensors_io import SafetensorsFile


def _storage_dtype(dtype: torch.dtype, integer: bool) -> torch.dtype:
    if dtype in (torch.float32, torch.float64):
        return torch.float32
    if dtype in (torch.bfloat16, torch.float16):
        return dtype
    if dtype in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool):
        return torch.int32
    raise EngineError(f"unsupported tensor dtype {dtype}", code="invalid_dtype")


class WeightStore:
    """Tensors by name on one device."""

    def __init__(self, tensors: dict[str, torch.Tensor], device: torch.device | str = "cpu"):
        self.device = torch.device(device)
        self._tensors = tensors

    # --- loading ----------------------------------------------------------------------
    @classmethod
    def load(cls, model_dir: str | Path, expected: Iterable[TensorSpec], device: torch.device | str = "cpu") -> "WeightStore":
        model_dir = Path(model_dir)
        files = _weight_files(model_dir)
        expected = list(expected)
        found: dict[str, SafetensorsFile] = {}
        for file in files:
            for name in file.names():
                if name in found:
                    raise WeightError(f"tensor {name!r} appears in more than one weight file", code="invalid_format")
                found[name] = file
        by_name = {spec.name: spec for spec in expected}
        missing = [s.name for s in expected if s.name not in found and not s.optional]
        unexpected = sorted(name for name in found if name not in by_name)
        wrong = []
        for spec in expected:
            if spec.name in found:
                shape = found[spec.name].shape(spec.name)
                if tuple(shape) != tuple(spec.shape):
                    wrong.append(f"{spec.name}: file has {list(shape)}, model needs {list(spec.shape)}")
        if missing or unexpected or wrong:
            parts = [f"weights in {model_dir} do not fit the model"]
            if missing:
                parts.append(f"missing ({len(missing)}): " + ", ".join(missing))
            if unexpected:
                parts.append(f"unexpected ({len(unexpected)}): " + ", ".join(unexpected))
            if wrong:
                parts.append(f"wrong shape ({len(wrong)}): " + "; ".join(wrong))
            raise WeightError(". ".join(parts))
        tensors: dict[str, torch.Tensor] = {}
        device = torch.device(device)
        for spec in expected:
            if spec.name not in found:
                continue
            raw = found[spec.name].tensor(spec.name)
            target = _storage_dtype(raw.dtype, spec.integer)
            tensors[spec.name] = raw.to(device=device, dtype=target, copy=True)
        for file in files:
            file.close()
        return cls(tensors, device)

    # --- lookup -----------------------------------------------------------------------
    def has(self, name: str) -> bool:
        return name in self._tensors

    def names(self) -> list[str]:
        return list(self._tensors)

    def get(self, name: str, dtype: torch.dtype | None = None) -> torch.Tensor:
        """The stored tensor, or a copy in ``dtype`` when that differs from how it is stored."""
        try:
            tensor = self._tensors[name]
        except KeyError:
            raise WeightError(f"required tensor is missing: {name}") from None
        if dtype is not None and tensor.dtype != dtype:
            tensor = tensor.to(dtype)
        return tensor

    def release(self, name: str) -> None:
        """Drop the store's reference once a part holds its own (fused or cast) copy."""
        self._tensors.pop(name, None)


def _weight_files(model_dir: Path) -> list[SafetensorsFile]:
    index = model_dir / "model.safetensors.index.json"
    single = model_dir / "model.safetensors"
    if single.exists():
        return [SafetensorsFile(single)]
    if index.exists():
        try:
            weight_map = json.loads(index.read_text())["weight_map"]
        except (OSError, KeyError, json.JSONDecodeError) as exc:
            raise WeightError(f"malformed {index}", code="invalid_format") from exc
        return [SafetensorsFile(model_dir / shard) for shard in sorted(set(weight_map.values()))]
    raise EngineError(f"no model.safetensors in {model_dir}", code="io")
