#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at TinyLlama-1.1B shapes with random weights, on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl engine|reference]

One JSON line on standard output.  A "step" is one decode step of the whole batch.
  value      decoded tokens per second, timed on the device with CUDA events around K replays of
             the decode step (forward, sampling and advancing on the device, no host round trip);
  e2e        the same through the Python entry point (Engine.step): every step copies the input
             token ids from pinned host memory and reads the sampled ids back;
  prefill    one 2,048-token prompt through the step function, with the fraction of the tensor peak;
  roofline   bytes a decode step must read (every weight once + the cache of the live requests)
             divided by its time, against the measured copy bandwidth;
  points     decode tokens per second at batch 1 and 64.
Between timed steps no cache flush is needed: a step reads about 2 GB of weights, far more than
the 126 MB L2, so nothing survives from one step to the next.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# BASELINE.json configs[2]: TinyLlama 1.1B shapes
SHAPES = dict(hidden_size=2048, intermediate_size=5632, num_hidden_layers=22, num_attention_heads=32, num_key_value_heads=4,
              max_position_embeddings=2048, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0)
PROMPT_TOKENS = 1024
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            flat = {}

            def walk(node):
                if isinstance(node, dict):
                    for key, value in node.items():
                        if isinstance(value, (int, float)) and key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                            flat.setdefault(key, float(value))
                        else:
                            walk(value)
                elif isinstance(node, list):
                    for value in node:
                        walk(value)

            walk(data)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return flat, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons while a timed region runs (NVML reads only; nvidia-smi as a fallback)."""

    QUERY = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self):
        self.clocks: list[int] = []
        self.max_clock = None
        self.reasons: set[str] = set()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._nvml = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(0)
            self.max_clock = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001
            self._nvml = None

    def _sample_nvml(self) -> None:
        nv = self._nvml
        self.clocks.append(int(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)))
        try:
            mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
        except Exception:  # noqa: BLE001
            mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
        self.reasons |= {name for name, bit in self.REASONS.items() if mask & bit}

    def _sample_smi(self) -> None:
        out = subprocess.run(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits"],
                             capture_output=True, text=True, timeout=5).stdout.strip()
        if out:
            cells = [c.strip() for c in out.splitlines()[0].split(",")]
            if cells[0].isdigit():
                self.clocks.append(int(cells[0]))
            if cells[1].isdigit():
                self.max_clock = int(cells[1])
            self.reasons |= {name for name, flag in zip(self.REASONS, cells[2:6]) if flag.lower().startswith("active")}

    def _run(self):
        while not self._stop.is_set():
            try:
                self._sample_nvml() if self._nvml is not None else self._sample_smi()
            except Exception:  # noqa: BLE001
                return
            self._stop.wait(0.01 if self._nvml is not None else 0.2)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        clocks = sorted(self.clocks)
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": self.max_clock, "reasons": sorted(self.reasons), "samples": len(clocks)}


def model_folder(layers: int) -> Path:
    """A random-weights model folder at the benchmark shapes (kept in the temporary folder between runs)."""
    from tinyllama_inference_engine_b200.weights import write_random_model

    folder = Path(tempfile.gettempdir()) / f"tlie_b200_bench_{os.getuid()}_L{layers}"
    if not (folder / "model.safetensors").exists():
        staging = Path(tempfile.mkdtemp(prefix="tlie_b200_bench_", dir=tempfile.gettempdir()))
        write_random_model(staging, dict(SHAPES, num_hidden_layers=layers), seed=0)
        try:
            os.replace(staging, folder)
        except OSError:
            return staging if not (folder / "model.safetensors").exists() else folder
    return folder


def decode_bytes(layers: int, batch: int, mean_context: float) -> float:
    """Bytes one decode step must read: every weight once, and the keys and values of the live requests."""
    h, i, v = SHAPES["hidden_size"], SHAPES["intermediate_size"], SHAPES["vocab_size"]
    d = h // SHAPES["num_attention_heads"]
    kv = SHAPES["num_key_value_heads"] * d
    per_layer = (h * (h + 2 * kv) + h * h + 2 * i * h + h * i) * 2 + 2 * h * 4
    weights = layers * per_layer + v * h * 2 + h * 4
    cache = batch * mean_context * layers * 2 * kv * 2
    return weights + cache


def prefill_flops(layers: int, tokens: int) -> float:
    h, i, v = SHAPES["hidden_size"], SHAPES["intermediate_size"], SHAPES["vocab_size"]
    d = h // SHAPES["num_attention_heads"]
    kv = SHAPES["num_key_value_heads"] * d
    linear = 2.0 * tokens * (h * (h + 2 * kv) + h * h + 2 * i * h + h * i) * layers + 2.0 * v * h
    attention = 4.0 * SHAPES["num_attention_heads"] * d * tokens * (tokens + 1) / 2 * layers
    return linear + attention


def run_engine(args) -> dict:
    import numpy as np
    import torch

    from tinyllama_inference_engine_b200 import EngineConfig, ops
    from tinyllama_inference_engine_b200.engine.api import Engine
    from tinyllama_inference_engine_b200.engine.batch import StepEntry
    from tinyllama_inference_engine_b200.engine.decode_session import DecodeSession
    from tinyllama_inference_engine_b200.engine.request import SamplingParams
    from tinyllama_inference_engine_b200.ops import fast

    layers, steps, warmup = args.layers, args.steps, args.warmup
    folder = model_folder(layers)
    rng = np.random.default_rng(0)
    vocab = SHAPES["vocab_size"]
    generated = warmup + steps + 8   # requests whose prompts ran in different steps are a few tokens apart: none finishes inside the timed steps
    if PROMPT_TOKENS + generated > SHAPES["max_position_embeddings"]:
        raise SystemExit("warmup + steps must stay within the 2,048-token context after a 1,024-token prompt")

    def prompts(count, length):
        return [[int(t) for t in rng.integers(0, vocab, size=length)] for _ in range(count)]

    def event_ms(fn) -> float:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end)

    largest = max(64, args.batch)
    config = EngineConfig(dtype="bfloat16", page_size=64, max_cache_tokens=largest * (PROMPT_TOKENS + 64 * (-(-generated // 64)) + 64),
                          max_requests=largest, max_batch_tokens=PREFILL_TOKENS)
    engine = Engine(folder, config)
    runner = engine.runner

    library_per_step: dict[int, int] = {}

    def device_decode(batch: int) -> tuple[float, float, int, dict]:
        """Tokens per second of K decode steps kept on the device; also ms per step, kernels per step, clocks."""
        ids = [f"d{batch}-{i}" for i in range(batch)]
        for rid, prompt in zip(ids, prompts(batch, PROMPT_TOKENS)):
            runner.step([StepEntry(rid, prompt, [])])
        session = DecodeSession(runner, batch)
        session.load(ids, [int(t) for t in rng.integers(0, vocab, size=batch)], [SamplingParams()] * batch, [0] * batch)
        for _ in range(max(warmup, 3)):
            session.step()
        with ClockSampler() as clocks:
            ms = event_ms(lambda: [session.step() for _ in range(steps)])
        for rid in ids:
            runner.finish(rid)
        library_per_step[batch] = session.library_calls_per_step
        return batch * steps / (ms / 1e3), ms / steps, session.kernels_per_step, clocks.summary()

    sections = set(args.sections.split(","))
    value, ms_per_step, kernels_per_step, clocks = device_decode(args.batch) if "decode" in sections else (0.0, 1.0, 0, {})
    first_context = PROMPT_TOKENS + max(warmup, 3)
    mean_context = first_context + (steps + 1) / 2.0
    step_bytes = decode_bytes(layers, args.batch, mean_context)
    peak, peak_kind = peaks()
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9

    # the same through the Python entry point: host token ids in, sampled ids out, every step
    e2e = None
    if "e2e" in sections:
        ids = [engine.add_request(p, SamplingParams(max_tokens=generated)) for p in prompts(args.batch, PROMPT_TOKENS)]
        while any(not engine.requests[i].generated for i in ids):
            engine.step()
        for _ in range(max(warmup, 3)):
            engine.step()
        torch.cuda.synchronize()
        started = time.perf_counter()
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
        e2e_seconds = time.perf_counter() - started
        for i in ids:
            engine.cancel(i)
        e2e = {"value": args.batch * steps / e2e_seconds, "unit": "tokens/s", "h2d_bytes_per_step": args.batch * 4, "d2h_bytes_per_step": args.batch * 4}

    # prefill of one 2,048-token prompt
    prefill = None
    if "prefill" in sections:
        prefill_ms = []
        for index, prompt in enumerate(prompts(3 + args.prefill_samples, PREFILL_TOKENS)):
            rid = f"p{index}"
            prefill_ms.append(event_ms(lambda: runner.step([StepEntry(rid, prompt, [PREFILL_TOKENS - 1])])))
            runner.finish(rid)
        timed = sorted(prefill_ms[3:])
        best = timed[len(timed) // 2]
        flops = prefill_flops(layers, PREFILL_TOKENS)
        prefill = {"value": PREFILL_TOKENS / (best / 1e3), "tokens": PREFILL_TOKENS, "ms": best,
                   "frac": flops / (best / 1e3) / (peak["bf16_tflops"] * 1e12), "tflops": flops / (best / 1e3) / 1e12}

    points = {}
    if "points" in sections:
        for batch in (1, 64):
            points[f"decode_b{batch}"] = value if batch == args.batch else device_decode(batch)[0]

    full_layers = SHAPES["num_hidden_layers"]
    return {
        "metric": "decode tokens/s at batch 8 (TinyLlama 1.1B shapes, 1,024-token prompts)" if args.batch == 8 else f"decode tokens/s at batch {args.batch}",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights N(0, 0.02), uniform random token ids)",
        "impl": "engine",
        "config": {"model": "TinyLlama-1.1B shapes", "layers": layers, "layers_of_model": full_layers, "hidden": SHAPES["hidden_size"],
                   "heads": SHAPES["num_attention_heads"], "kv_heads": SHAPES["num_key_value_heads"], "head_dim": 64,
                   "intermediate": SHAPES["intermediate_size"], "vocab": vocab, "global_batch": args.batch, "seq_len": SHAPES["max_position_embeddings"],
                   "prompt_tokens": PROMPT_TOKENS, "context_first_timed_step": first_context, "page_size": 64, "parallelism": "single GPU",
                   "l2": "inputs larger than L2: each step streams ~2 GB of weights", "peaks": peak_kind},
        "e2e": e2e,
        "gpu_launches": kernels_per_step * steps,
        "library_gemms_per_step": library_per_step.get(args.batch, 0),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s", "frac": achieved / peak["hbm_gbs"], "bytes_per_step": step_bytes},
        "points": points,
        "clocks": clocks,
    }


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=SHAPES["num_hidden_layers"])
    parser.add_argument("--prefill-samples", type=int, default=5)
    parser.add_argument("--impl", default="engine", choices=["engine", "reference"])
    parser.add_argument("--sections", default="decode,e2e,prefill,points", help="which measurements to take (all by default; fewer for profiling runs)")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: this engine is single-GPU by design (asked for {args.gpus})")
        return 2
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    print(json.dumps(run_engine(args)))
    return 0


REFERENCE_UNAVAILABLE = ("pip install --no-deps of the reference yields metadata only (it ships no Python package); its engine is a CMake CUDA binary "
                         "that fetches SentencePiece and cpp-httplib from the network at configure time and loads only the SHA-256-pinned "
                         "TinyLlama-1.1B-Chat checkpoint and tokenizer, none of which exist offline")

if __name__ == "__main__":
    sys.exit(main())
