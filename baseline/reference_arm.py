"""The reference arm of bench.py: the unmodified reference engine, timed on the same metric and shapes.

The reference ships no Python package (``pip install --target baseline/_ref`` leaves metadata only); its engine is C++ and
CUDA.  So the arm keeps a copy of the reference's source tree under ``baseline/_ref`` (``src/``, ``include/``, ``scripts/``),
compiles its unmodified ``src/{error,sha256,model_config,weight_store,operators}.cpp`` and
``src/cuda/{kernels.cu,model.cu,weight_store.cpp}`` with nvcc and cuBLAS for this GPU, links them with
``baseline/reference_driver.cu`` (a benchmark loop in the manner of the reference's ``app/batch_benchmark.cu:67-114``), and
runs that program.  Nothing of this repository's engine, kernels or loaders is on that path:

* weights: the random values of the benchmark's model folder, converted to the reference's float16 TLIEWGT container by the
  reference's own writer (``scripts/tlie_format.py:25-75``); the loader's two SHA-256 pins are options of the call
  (``src/cuda/weight_store.cpp:175-219``) and are given the file's own digests;
* configuration: a config.json with exactly the TinyLlama-1.1B values the reference demands (``src/model_config.cpp:54-76``),
  read by ``ModelConfig::Load``;
* model: ``TinyLlamaCuda::Create`` / ``ForwardBatch`` / ``Reset`` and host-side ``GreedySample``, as the reference's own
  programs use them.  ``value`` is the device time the reference measures itself (``CudaStepTimings::compute_ms``), ``e2e``
  the host clock around a whole step (token ids in, float16 logits of every row out and converted, greedy on the host).
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"
SOURCES = ["src/error.cpp", "src/sha256.cpp", "src/model_config.cpp", "src/weight_store.cpp", "src/operators.cpp",
           "src/cuda/kernels.cu", "src/cuda/model.cu", "src/cuda/weight_store.cpp"]
# what ModelConfig::ValidateFixedTinyLlama accepts, and nothing else (src/model_config.cpp:54-76)
PINNED_CONFIG = {"model_type": "llama", "hidden_size": 2048, "intermediate_size": 5632, "num_hidden_layers": 22, "num_attention_heads": 32,
                 "num_key_value_heads": 4, "max_position_embeddings": 2048, "vocab_size": 32000, "bos_token_id": 1, "eos_token_id": 2,
                 "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "attention_bias": False, "tie_word_embeddings": False, "hidden_act": "silu",
                 "torch_dtype": "bfloat16"}


class Unavailable(Exception):
    """The reference cannot be built or run here; the message is the one-line reason."""


def ensure_sources() -> None:
    """``baseline/_ref`` holds the reference's tree; fill it from a checkout if it is empty and one is at hand."""
    if all((REF / s).exists() for s in SOURCES):
        return
    origin = Path(os.environ.get("TLIE_REFERENCE_SOURCE", str(HERE.parent.parent / "reference")))   # a checkout beside this repository
    if not (origin / "src" / "cuda" / "model.cu").exists():
        raise Unavailable(f"no copy of the reference's sources under {REF} and none at {origin}")
    REF.mkdir(parents=True, exist_ok=True)
    for name in ("src", "include", "scripts", "LICENSE"):
        source = origin / name
        target = REF / name
        if source.is_dir():
            shutil.copytree(source, target, dirs_exist_ok=True)
        elif source.exists():
            shutil.copy2(source, target)


def _json_include() -> Path:
    """A folder that holds nlohmann/json.hpp (src/model_config.cpp includes it; the reference fetches it with CMake)."""
    roots = [Path(p) for p in sys.path if p and "site-packages" in p] + [Path("/usr/include"), Path("/usr/local/include")]
    for root in roots:
        if (root / "nlohmann" / "json.hpp").exists():
            return root
        for found in root.glob("**/nlohmann/json.hpp"):
            return found.parent.parent
    raise Unavailable("nlohmann/json.hpp, which the reference's src/model_config.cpp includes, was not found on this machine")


def build() -> Path:
    """Compile the reference with the driver; returns the program's path (cached by a digest of every source)."""
    ensure_sources()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise Unavailable("nvcc was not found")
    digest = hashlib.sha1()
    for path in [HERE / "reference_driver.cu"] + [REF / s for s in SOURCES] + sorted((REF / "include").rglob("*.hpp")):
        digest.update(path.read_bytes())
    out = REF / "_build"
    out.mkdir(parents=True, exist_ok=True)
    program = out / f"reference_driver_{digest.hexdigest()[:12]}"
    if program.exists():
        return program
    # the reference's own flags (CMakeLists.txt:123-135: C++20, release, -lineinfo, --expt-relaxed-constexpr), for this GPU
    command = [nvcc, "-std=c++20", "-O3", "-lineinfo", "--expt-relaxed-constexpr", "-gencode", "arch=compute_100,code=sm_100",
               "-I", str(REF / "include"), "-I", str(_json_include()), str(HERE / "reference_driver.cu"), *[str(REF / s) for s in SOURCES],
               "-lcublas", "-o", str(program) + ".partial"]
    print("[reference arm] compiling the reference for sm_100 ...", file=sys.stderr, flush=True)
    done = subprocess.run(command, capture_output=True, text=True)
    if done.returncode != 0:
        raise Unavailable("nvcc failed on the reference's sources: " + (done.stderr.strip().splitlines() or ["no message"])[-1][:300])
    os.replace(str(program) + ".partial", program)
    return program


def _sha256(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as file:
        while chunk := file.read(1 << 24):
            h.update(chunk)
    return h.hexdigest()


def convert_weights(model_folder: Path) -> tuple[Path, Path, str, str]:
    """The model folder's tensors as the reference's float16 container: (config.json, weights, file digest, source digest)."""
    ensure_sources()
    import numpy as np

    sys.path.insert(0, str(REF / "scripts"))
    try:
        from tlie_format import write_tensor_file   # the reference's own writer
    finally:
        sys.path.pop(0)
    folder = Path(tempfile.gettempdir()) / f"tlie_b200_reference_{os.getuid()}"
    folder.mkdir(parents=True, exist_ok=True)
    source_digest = _sha256(Path(model_folder) / "model.safetensors")
    weights, stamp = folder / "model-fp16.tliewgt", folder / "model-fp16.json"
    (folder / "config.json").write_text(json.dumps(PINNED_CONFIG))
    if weights.exists() and stamp.exists():
        recorded = json.loads(stamp.read_text())
        if recorded.get("source") == source_digest:
            return folder / "config.json", weights, recorded["file"], source_digest
    raw = np.memmap(Path(model_folder) / "model.safetensors", dtype=np.uint8, mode="r")
    n = int.from_bytes(raw[:8].tobytes(), "little")
    header = {k: v for k, v in json.loads(raw[8 : 8 + n].tobytes()).items() if k != "__metadata__"}

    def tensors():
        for name, info in header.items():
            begin, end = info["data_offsets"]
            blob = np.array(raw[8 + n + begin : 8 + n + end])
            if info["dtype"] == "BF16":
                value = (blob.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
            else:
                value = blob.view({"F32": np.float32, "F16": np.float16}[info["dtype"]]).astype(np.float32)
            yield name, value.reshape(info["shape"])

    print("[reference arm] writing the weights as float16 TLIEWGT with the reference's writer ...", file=sys.stderr, flush=True)
    write_tensor_file(weights, source_digest, tensors(), len(header), "float16")
    file_digest = _sha256(weights)
    stamp.write_text(json.dumps({"source": source_digest, "file": file_digest}))
    return folder / "config.json", weights, file_digest, source_digest


def run(model_folder: Path, prompt_tokens: int, warmup: int, steps: int, batches: list[int]) -> dict[int, dict]:
    """Run the reference's decode steps; per batch size the driver's record (device / transfer / wall ms per step)."""
    program = build()
    config, weights, file_digest, source_digest = convert_weights(model_folder)
    command = [str(program), str(config), str(weights), file_digest, source_digest, str(prompt_tokens), str(warmup), str(steps), *map(str, batches)]
    print("[reference arm] running the reference: " + " ".join(command[5:]), file=sys.stderr, flush=True)
    done = subprocess.run(command, capture_output=True, text=True)
    if done.returncode != 0:
        raise Unavailable("the reference's program failed: " + (done.stderr.strip().splitlines() or [f"exit code {done.returncode}"])[-1][:300])
    records = {}
    for line in done.stdout.splitlines():
        if line.startswith("{"):
            record = json.loads(line)
            records[int(record["batch"])] = record
    if set(records) != set(batches):
        raise Unavailable("the reference's program did not report every batch size")
    return records
