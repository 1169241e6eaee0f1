"""SHA-256 of a model folder's weight files, and the check against a pinned digest.

The reference pins its checkpoints by digest: the loader takes ``expected_file_sha256`` and refuses a file whose digest differs
with ``checksum_mismatch`` (include/tlie/weight_store.hpp:30-34, src/weight_store.cpp:150-190, include/tlie/sha256.hpp:14-32).
Here the pin is an option of the engine (``EngineConfig.weights_sha256``, ``--weights-sha256`` on the command line); nothing is
pinned by default, since this engine loads any checkpoint of the architecture.  A folder with one ``model.safetensors`` is pinned
by that file's digest; a sharded one by the digest of its shards' digests in the order of their names.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

from ..errors import EngineError


def file_sha256(path: str | Path) -> str:
    digest = hashlib.sha256()
    try:
        with open(path, "rb") as file:
            while chunk := file.read(1 << 24):
                digest.update(chunk)
    except OSError as exc:
        raise EngineError(f"unable to read {path}: {exc}", code="io") from exc
    return digest.hexdigest()


def weights_sha256(model_dir: str | Path) -> str:
    """The digest that pins the weights of ``model_dir`` (see the module's text)."""
    model_dir = Path(model_dir)
    single = model_dir / "model.safetensors"
    if single.exists():
        return file_sha256(single)
    index = model_dir / "model.safetensors.index.json"
    if not index.exists():
        raise EngineError(f"no model.safetensors in {model_dir}", code="io")
    try:
        shards = sorted(set(json.loads(index.read_text())["weight_map"].values()))
    except (OSError, KeyError, json.JSONDecodeError) as exc:
        raise EngineError(f"malformed {index}", code="invalid_format") from exc
    combined = hashlib.sha256()
    for shard in shards:
        combined.update(bytes.fromhex(file_sha256(model_dir / shard)))
    return combined.hexdigest()


def parse_sha256(text: str) -> str:
    """64 hexadecimal digits, lower case (include/tlie/sha256.hpp:32)."""
    cleaned = text.strip().lower()
    if len(cleaned) != 64 or any(c not in "0123456789abcdef" for c in cleaned):
        raise EngineError("a SHA-256 digest is 64 hexadecimal digits", code="invalid_argument")
    return cleaned


def verify_weights(model_dir: str | Path, expected: str) -> str:
    """Raises ``checksum_mismatch`` unless the folder's weights have the digest ``expected``; returns the digest."""
    wanted = parse_sha256(expected)
    found = weights_sha256(model_dir)
    if found != wanted:
        raise EngineError(f"weights in {model_dir} have SHA-256 {found}, expected {wanted}", code="checksum_mismatch")
    return found
