"""Reading and writing the safetensors container, by tensor name.

Layout of a file: an unsigned 64-bit little-endian header length, a JSON header
mapping each tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}``
(offsets relative to the end of the header), then the raw little-endian payload.
The reference never reads this format in C++; its Python converters open it with
``safe_open(...).get_tensor(name)`` (scripts/convert_model.py:23-27).  The payload is
memory-mapped and every offset is checked against the file before it is used.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch

from ..errors import EngineError, FormatError

_DTYPES = {
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F32": (torch.float32, 4),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {dtype: name for name, (dtype, _) in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


class SafetensorsFile:
    """A memory-mapped safetensors file; ``tensor(name)`` returns a read-only view."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        try:
            self._file = open(self.path, "rb")
        except OSError as exc:
            raise EngineError(f"unable to open weight file: {self.path}", code="io") from exc
        size = self.path.stat().st_size
        if size < 8:
            raise FormatError(f"{self.path}: truncated, no header length")
        (header_len,) = struct.unpack("<Q", self._file.read(8))
        if header_len > _MAX_HEADER or 8 + header_len > size:
            raise FormatError(f"{self.path}: header length {header_len} exceeds the file")
        try:
            header = json.loads(self._file.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise FormatError(f"{self.path}: malformed JSON header: {exc}") from exc
        if not isinstance(header, dict):
            raise FormatError(f"{self.path}: header is not a JSON object")
        self.metadata = header.pop("__metadata__", {})
        self._data_start = 8 + header_len
        payload = size - self._data_start
        self.entries: dict[str, tuple[str, tuple[int, ...], int, int]] = {}
        spans = []
        for name, info in header.items():
            try:
                dtype, shape, (begin, end) = info["dtype"], tuple(info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError) as exc:
                raise FormatError(f"{self.path}: bad header entry for {name!r}") from exc
            if dtype not in _DTYPES:
                raise EngineError(f"{self.path}: tensor {name!r} has unsupported dtype {dtype}", code="invalid_dtype")
            count = 1
            for dim in shape:
                if not isinstance(dim, int) or dim < 0:
                    raise FormatError(f"{self.path}: tensor {name!r} has a bad shape {shape}")
                count *= dim
            if not (0 <= begin <= end <= payload):
                raise FormatError(f"{self.path}: tensor {name!r} lies outside the file (truncated?)")
            if end - begin != count * _DTYPES[dtype][1]:
                raise FormatError(
                    f"{self.path}: tensor {name!r} holds {end - begin} bytes, its shape needs {count * _DTYPES[dtype][1]}"
                )
            self.entries[name] = (dtype, shape, begin, end)
            spans.append((begin, end, name))
        spans.sort()
        for (_, end_a, name_a), (begin_b, _, name_b) in zip(spans, spans[1:]):
            if begin_b < end_a:
                raise FormatError(f"{self.path}: tensors {name_a!r} and {name_b!r} overlap")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> list[str]:
        return list(self.entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name][0]][0]

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, begin, end = self.entries[name]
        torch_dtype = _DTYPES[dtype][0]
        if end == begin:
            return torch.empty(shape, dtype=torch_dtype)
        view = memoryview(self._map)[self._data_start + begin : self._data_start + end]
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the mapping is read-only; the view is only copied from
            flat = torch.frombuffer(view, dtype=torch_dtype)
        return flat.reshape(shape)

    def close(self) -> None:
        self._map = None
        self._file.close()


def write_safetensors(path: str | Path, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Write tensors (in the given order) as one safetensors file."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, tensor in tensors.items():
        tensor = tensor.detach().cpu().contiguous()
        if tensor.dtype not in _NAMES:
            raise EngineError(f"cannot store dtype {tensor.dtype} for {name!r}", code="invalid_dtype")
        raw = tensor.view(torch.uint8).numpy().tobytes() if tensor.numel() else b""
        header[name] = {
            "dtype": _NAMES[tensor.dtype],
            "shape": list(tensor.shape),
            "data_offsets": [offset, offset + len(raw)],
        }
        offset += len(raw)
        blobs.append(raw)
    encoded = json.dumps(header, separators=(",", ":")).encode("utf-8")
    encoded += b" " * ((8 - len(encoded) % 8) % 8)
    with open(path, "wb") as out:
        out.write(struct.pack("<Q", len(encoded)))
        out.write(encoded)
        for raw in blobs:
            out.write(raw)
