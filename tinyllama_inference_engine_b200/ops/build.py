"""Compiling the CUDA sources for sm_100a and loading them.

The kernels are plain CUDA with ``extern "C"`` launchers, so they are compiled with
``nvcc`` directly (no binding generator, seconds per file) into one shared library
per *kernel set* and loaded with ``ctypes``.  A set is a list of source files plus
preprocessor definitions (for instance the head size a tensor-core kernel is
specialised for), so a process compiles only what its model needs.  Libraries are
cached by a hash of their sources and flags in ``csrc/_build`` inside the package
(or, where that is not writable, in a per-user temporary folder).
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

from ..errors import KernelError

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def _nvcc() -> str:
    for candidate in (os.environ.get("TLIE_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise KernelError("nvcc was not found; the CUDA kernels of this engine cannot be built")


def build_dir() -> Path:
    override = os.environ.get("TLIE_B200_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates.append(CSRC / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"tlie_b200_build_{os.getuid()}")
    for folder in candidates:
        try:
            folder.mkdir(parents=True, exist_ok=True)
            with tempfile.NamedTemporaryFile(prefix=".probe_", dir=folder):   # a name of its own: threads and processes may ask at once
                pass
            return folder
        except OSError:
            continue
    raise KernelError("no writable folder for compiled kernels (set TLIE_B200_BUILD_DIR)")


def _digest(sources: list[Path], flags: list[str]) -> str:
    h = hashlib.sha1()
    for path in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + list(sources):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


class _Progress:
    """Prints a line now and then while a compilation runs."""

    def __init__(self, what: str):
        self.what = what
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self) -> None:
        start = time.time()
        while not self._stop.wait(10.0):
            print(f"[tlie-b200] still compiling {self.what} ({time.time() - start:.0f} s)", file=sys.stderr, flush=True)

    def __enter__(self):
        print(f"[tlie-b200] compiling {self.what} for sm_100a ...", file=sys.stderr, flush=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join()


def library_path(name: str, sources: list[str], defines: dict[str, object] | None = None) -> tuple[Path, list[Path], list[str]]:
    paths = [CSRC / s for s in sources]
    flags = ARCH_FLAGS + BASE_FLAGS + [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
    return build_dir() / f"lib{name}_{_digest(paths, flags)}.so", paths, flags


def build_library(name: str, sources: list[str], defines: dict[str, object] | None = None, extra_link: list[str] | None = None) -> Path:
    """Compile ``sources`` (file names under csrc/) into a shared library; return its path."""
    target, paths, flags = library_path(name, sources, defines)
    if target.exists():
        return target
    nvcc = _nvcc()
    work = Path(tempfile.mkdtemp(prefix=f"{name}_", dir=target.parent))
    try:
        with _Progress(f"{name} ({len(paths)} files)"):
            def compile_one(path: Path) -> Path:
                obj = work / (path.stem + ".o")
                cmd = [nvcc, *flags, "-I", str(CSRC), "-c", str(path), "-o", str(obj)]
                done = subprocess.run(cmd, capture_output=True, text=True)
                if done.returncode != 0:
                    raise KernelError(f"nvcc failed for {path.name}:\n{done.stdout}\n{done.stderr}")
                return obj

            with ThreadPoolExecutor(max_workers=min(8, len(paths))) as pool:
                objects = list(pool.map(compile_one, paths))
            staged = work / target.name
            link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(staged), *map(str, objects), *(extra_link or [])]
            done = subprocess.run(link, capture_output=True, text=True)
            if done.returncode != 0:
                raise KernelError(f"linking {target.name} failed:\n{done.stdout}\n{done.stderr}")
            os.replace(staged, target)  # atomic: concurrent builders cannot see a partial file
    finally:
        shutil.rmtree(work, ignore_errors=True)
    return target


def load_library(name: str, sources: list[str], defines: dict[str, object] | None = None, extra_link: list[str] | None = None) -> ctypes.CDLL:
    key = name if not defines else name + repr(sorted(defines.items()))
    found = _loaded.get(key)   # every kernel launch comes through here: no lock and no string building once it is loaded
    if found is not None:
        return found
    with _lock:
        if key not in _loaded:
            path = build_library(name, sources, defines, extra_link)
            try:
                _loaded[key] = ctypes.CDLL(str(path))
            except OSError as exc:
                raise KernelError(f"cannot load {path}: {exc}") from exc
        return _loaded[key]
