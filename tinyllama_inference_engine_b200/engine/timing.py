"""What a step cost, split as the reference splits it, and optional profiler ranges.

``StepTimings`` has the fields of the reference's ``CudaStepTimings`` (include/tlie/cuda/model.hpp:14-18): device time of
the forward pass, device time of the copies around it, and host wall time of the whole call, taken with CUDA events on
the step's stream as the reference does (src/cuda/model.cu:380-385, 512-526).  Asking for timings makes the call wait
for the device at its end; a step that is not asked costs nothing extra.

``nvtx_range`` marks prefill, decode and sampling for a profiler's timeline as the reference's program does
(app/cuda_reference.cu:31-37); it is a no-op unless ranges were switched on.
"""
from __future__ import annotations

import contextlib
import os
import time
from dataclasses import dataclass

import torch


@dataclass
class StepTimings:
    compute_ms: float = 0.0      # the forward pass (and sampling where the step samples), on the device
    transfer_ms: float = 0.0     # copies between host and device that belong to the step, on the device
    wall_ms: float = 0.0         # the whole call, on the host's clock
    steps: int = 0

    def add(self, other: "StepTimings") -> None:
        self.compute_ms += other.compute_ms
        self.transfer_ms += other.transfer_ms
        self.wall_ms += other.wall_ms
        self.steps += max(1, other.steps)


class StepClock:
    """Events around the parts of one step; ``finish`` waits for the device and fills a StepTimings."""

    def __init__(self, device: torch.device, enabled: bool):
        self.enabled = enabled and device.type == "cuda"
        self._started = time.perf_counter() if enabled else 0.0
        self._marks: list = []
        if self.enabled:
            self.mark()

    def mark(self) -> None:
        if self.enabled:
            event = torch.cuda.Event(enable_timing=True)
            event.record()
            self._marks.append(event)

    def finish(self, timings: StepTimings | None, kinds: tuple[str, ...]) -> None:
        """``kinds[i]`` says what lies between mark i and mark i + 1: "compute" or "transfer"."""
        if timings is None:
            return
        if self.enabled:
            self._marks[-1].synchronize()
            for kind, begin, end in zip(kinds, self._marks, self._marks[1:]):
                elapsed = begin.elapsed_time(end)
                if kind == "compute":
                    timings.compute_ms += elapsed
                else:
                    timings.transfer_ms += elapsed
        timings.wall_ms += (time.perf_counter() - self._started) * 1e3
        timings.steps += 1


_nvtx_on = os.environ.get("TLIE_NVTX", "0") == "1"


def enable_nvtx(on: bool = True) -> None:
    global _nvtx_on
    _nvtx_on = bool(on)


@contextlib.contextmanager
def nvtx_range(name: str):
    if not _nvtx_on or not torch.cuda.is_available():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
