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


@pytest.fixture(params=["library", "own"], ids=["small products by the library", "own products from 128 rows"])
def product_thresholds(request, monkeypatch):
    """Small products, and those whose tiles would leave SMs idle, go to the library (it is faster there); the second run of a test
    that uses this fixture takes the conditions away, so that the engine's own tensor-core products (plain, gated, adding into the
    residual) are checked through the engine at the test's small sizes too."""
    if request.param == "own":
        from tinyllama_inference_engine_b200.ops import fast

        for name, value in (("TCGEN05_MIN_ROWS", 128), ("TCGEN05_GATED_MIN_ROWS", 128), ("OWN_PRODUCT_MIN_EFFICIENCY", 0.0), ("OWN_PRODUCT_MIN_FLOP", 0.0),
                            ("OWN_ADDING_MIN_FLOP", 0.0), ("PAIR_MIN_ROWS", 256)):   # pairs of SMs from 256 rows: their kernels too
            monkeypatch.setattr(fast, name, value)
    return request.param
