from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for entry in (str(ROOT), str(ROOT / "tests")):
    if entry not in sys.path:
        sys.path.insert(0, entry)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs the engine's kernels on a B200)")


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Random tiny checkpoints (config.json + model.safetensors) in a temporary folder, by name."""
    from tiny_configs import ALL
    from tinyllama_inference_engine_b200.weights import write_random_model

    base = tmp_path_factory.mktemp("models")
    return {key: write_random_model(base / key, config, seed) for key, (config, seed) in ALL.items()}
