#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at real Llama shapes with random weights, on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--config tinyllama|llama2-7b|llama3-8b] [--layers L]
                    [--impl engine|reference]

One JSON line on standard output.  A "step" is one decode step of the whole batch.
  value      decoded tokens per second, timed on the device with CUDA events around K replays of
             the decode step (forward, sampling and advancing on the device, no host round trip);
  e2e        the same through the Python entry point (Engine.step): every step copies the input
             token ids from pinned host memory and reads the sampled ids back;
  prefill    one prompt of the configuration's prefill length through the step function, with the fraction of the tensor peak;
  roofline   bytes a decode step must read (every weight once + the cache of the live requests)
             divided by its time, against the measured copy bandwidth;
  points     decode tokens per second at batch 1 and 64 (with the vendor-library products each ran on).
The default configuration is TinyLlama 1.1B with all of its layers.  The larger shapes may run with fewer layers than the
checkpoints have (--layers); ``config`` then names both numbers, and every byte and flop count is of the layers that ran.
Between timed steps no cache flush is needed: a step reads gigabytes of weights, far more than
the 126 MB L2, so nothing survives from one step to the next.
``--impl reference`` runs the unmodified reference engine on the same metric (baseline/reference_arm.py).
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

# The shapes the metric is quoted on (one table over sizes, as the reference's scripts/benchmark.py:32-36 has one over contexts):
# layer sizes of the checkpoint, the prompt length of the decode runs, the length of the timed prefill.
CONFIGS = {
    "tinyllama": dict(model="TinyLlama-1.1B shapes", prompt_tokens=1024, prefill_tokens=2048, default_layers=22,
                      shapes=dict(hidden_size=2048, intermediate_size=5632, num_hidden_layers=22, num_attention_heads=32, num_key_value_heads=4,
                                  max_position_embeddings=2048, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0)),
    "llama2-7b": dict(model="Llama-2-7B shapes", prompt_tokens=1024, prefill_tokens=2048, default_layers=8,
                      shapes=dict(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=32,
                                  max_position_embeddings=4096, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0)),
    "llama3-8b": dict(model="Llama-3-8B shapes", prompt_tokens=7168, prefill_tokens=8192, default_layers=8,
                      shapes=dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                                  max_position_embeddings=8192, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0)),
}
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


def model_folder(name: str, shapes: dict, layers: int) -> Path:
    """A random-weights model folder at the benchmark shapes (kept in the temporary folder between runs)."""
    from tinyllama_inference_engine_b200.weights import write_random_model

    suffix = "" if name == "tinyllama" else f"_{name}"
    folder = Path(tempfile.gettempdir()) / f"tlie_b200_bench_{os.getuid()}{suffix}_L{layers}"
    if not (folder / "model.safetensors").exists():
        staging = Path(tempfile.mkdtemp(prefix="tlie_b200_bench_", dir=tempfile.gettempdir()))
        write_random_model(staging, dict(shapes, num_hidden_layers=layers, architectures=["LlamaForCausalLM"], model_type="llama", bos_token_id=1, eos_token_id=2), seed=0)
        try:
            os.replace(staging, folder)
        except OSError:
            return staging if not (folder / "model.safetensors").exists() else folder
    return folder


def decode_bytes(shapes: dict, layers: int, batch: int, mean_context: float) -> float:
    """Bytes one decode step must read: every weight once, and the keys and values of the live requests."""
    h, i, v = shapes["hidden_size"], shapes["intermediate_size"], shapes["vocab_size"]
    d = h // shapes["num_attention_heads"]
    kv = shapes["num_key_value_heads"] * d
    per_layer = (h * (h + 2 * kv) + h * h + 2 * i * h + h * i) * 2 + 2 * h * 4
    weights = layers * per_layer + v * h * 2 + h * 4
    cache = batch * mean_context * layers * 2 * kv * 2
    return weights + cache


def prefill_flops(shapes: dict, layers: int, tokens: int) -> float:
    h, i, v = shapes["hidden_size"], shapes["intermediate_size"], shapes["vocab_size"]
    d = h // shapes["num_attention_heads"]
    kv = shapes["num_key_value_heads"] * d
    linear = 2.0 * tokens * (h * (h + 2 * kv) + h * h + 2 * i * h + h * i) * layers + 2.0 * v * h
    attention = 4.0 * shapes["num_attention_heads"] * d * tokens * (tokens + 1) / 2 * layers
    return linear + attention


def config_record(args, chosen: dict, layers: int, first_context: int, peak_kind: str) -> dict:
    """The sizes that were run, flat (nothing deeper survives in the record)."""
    shapes = chosen["shapes"]
    return {"model": chosen["model"], "layers": layers, "layers_of_model": shapes["num_hidden_layers"], "hidden": shapes["hidden_size"],
            "heads": shapes["num_attention_heads"], "kv_heads": shapes["num_key_value_heads"], "head_dim": shapes["hidden_size"] // shapes["num_attention_heads"],
            "intermediate": shapes["intermediate_size"], "vocab": shapes["vocab_size"], "global_batch": args.batch, "seq_len": shapes["max_position_embeddings"],
            "prompt_tokens": chosen["prompt_tokens"], "prefill_tokens": chosen["prefill_tokens"], "context_first_timed_step": first_context, "page_size": 64,
            "parallelism": "single GPU", "l2": "inputs larger than L2: each step streams gigabytes of weights", "peaks": peak_kind}


def metric_name(args, chosen: dict) -> str:
    if args.config == "tinyllama" and args.batch == 8:
        return "decode tokens/s at batch 8 (TinyLlama 1.1B shapes, 1,024-token prompts)"
    return f"decode tokens/s at batch {args.batch} ({chosen['model']}, {chosen['prompt_tokens']:,}-token prompts)"


def run_engine(args) -> dict:
    import numpy as np
    import torch

    from tinyllama_inference_engine_b200 import EngineConfig
    from tinyllama_inference_engine_b200.engine.api import Engine
    from tinyllama_inference_engine_b200.engine.batch import StepEntry
    from tinyllama_inference_engine_b200.engine.decode_session import DecodeSession
    from tinyllama_inference_engine_b200.engine.request import SamplingParams

    chosen = CONFIGS[args.config]
    shapes, prompt_tokens, prefill_tokens = chosen["shapes"], chosen["prompt_tokens"], chosen["prefill_tokens"]
    layers, steps, warmup = args.layers or chosen["default_layers"], args.steps, args.warmup
    folder = model_folder(args.config, shapes, layers)
    rng = np.random.default_rng(0)
    vocab = shapes["vocab_size"]
    generated = warmup + steps + 8   # requests whose prompts ran in different steps are a few tokens apart: none finishes inside the timed steps
    if prompt_tokens + generated > shapes["max_position_embeddings"]:
        raise SystemExit(f"warmup + steps must stay within the {shapes['max_position_embeddings']:,}-token context after a {prompt_tokens:,}-token prompt")

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

    sections = set(args.sections.split(","))
    largest = max(64 if "points" in sections else 1, args.batch)
    cache_tokens = largest * (prompt_tokens + 64 * (-(-generated // 64)) + 64)
    # Requests of mixed length for the scheduler (prompts uniform between 64 tokens and the context, cut into
    # portions under the token budget and interleaved with the other requests' decode steps); all of them fit the cache at once.
    mixed_count, mixed_out = 32, 64
    mixed_lengths = [int(n) for n in rng.integers(64, min(4096, shapes["max_position_embeddings"] - mixed_out - 1) + 1, size=mixed_count)]
    if "mixed" in sections:
        largest = max(largest, mixed_count)
        cache_tokens = max(cache_tokens, sum(64 * (-(-(n + mixed_out) // 64)) + 64 for n in mixed_lengths))
    config = EngineConfig(dtype="bfloat16", page_size=64, max_cache_tokens=cache_tokens, max_requests=largest, max_batch_tokens=max(prefill_tokens, prompt_tokens))
    engine = Engine(folder, config)
    runner = engine.runner

    library_per_step: dict[int, int] = {}

    def device_decode(batch: int) -> tuple[float, float, int, dict]:
        """Tokens per second of K decode steps kept on the device; also ms per step, kernels per step, clocks."""
        ids = [f"d{batch}-{i}" for i in range(batch)]
        for rid, prompt in zip(ids, prompts(batch, prompt_tokens)):
            runner.step([StepEntry(rid, prompt, [])])
        session = DecodeSession(runner, batch, publish=False)   # these steps stay on the device: nothing goes to host memory
        session.load(ids, [int(t) for t in rng.integers(0, vocab, size=batch)], [SamplingParams()] * batch, [0] * batch)
        for _ in range(max(warmup, 3)):
            session.step()
        with ClockSampler() as clocks:
            ms = event_ms(lambda: [session.step() for _ in range(steps)])
        for rid in ids:
            runner.finish(rid)
        library_per_step[batch] = session.library_calls_per_step
        return batch * steps / (ms / 1e3), ms / steps, session.kernels_per_step, clocks.summary()

    value, ms_per_step, kernels_per_step, clocks = device_decode(args.batch) if "decode" in sections else (0.0, 1.0, 0, {})
    first_context = prompt_tokens + max(warmup, 3)
    mean_context = first_context + (steps + 1) / 2.0
    step_bytes = decode_bytes(shapes, layers, args.batch, mean_context)
    peak, peak_kind = peaks()
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9

    # the same through the Python entry point: host token ids in, sampled ids out, every step
    e2e = None
    if "e2e" in sections:
        ids = [engine.add_request(p, SamplingParams(max_tokens=generated)) for p in prompts(args.batch, prompt_tokens)]
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
        e2e = {"value": args.batch * steps / e2e_seconds, "unit": "tokens/s", "h2d_bytes_per_step": args.batch * 4, "d2h_bytes_per_step": (args.batch + 2) * 4}   # ids in; ids, the device error word and the step number out

    # prefill of one prompt
    prefill = None
    if "prefill" in sections:
        prefill_ms = []
        for index, prompt in enumerate(prompts(3 + args.prefill_samples, prefill_tokens)):
            rid = f"p{index}"
            prefill_ms.append(event_ms(lambda: runner.step([StepEntry(rid, prompt, [prefill_tokens - 1])])))
            runner.finish(rid)
        timed = sorted(prefill_ms[3:])
        best = timed[len(timed) // 2]
        flops = prefill_flops(shapes, layers, prefill_tokens)
        prefill = {"value": prefill_tokens / (best / 1e3), "tokens": prefill_tokens, "ms": best,
                   "frac": flops / (best / 1e3) / (peak["bf16_tflops"] * 1e12), "tflops": flops / (best / 1e3) / 1e12}

    points = {}
    if "points" in sections:
        for batch in (1, 64):
            if batch == args.batch:
                points[f"decode_b{batch}"] = value
                points[f"decode_b{batch}_hbm_frac"] = achieved / peak["hbm_gbs"]
            else:
                tokens_per_s, ms, _, _ = device_decode(batch)
                points[f"decode_b{batch}"] = tokens_per_s
                points[f"decode_b{batch}_hbm_frac"] = decode_bytes(shapes, layers, batch, mean_context) / (ms / 1e3) / 1e9 / peak["hbm_gbs"]
            points[f"decode_b{batch}_library_gemms_per_step"] = library_per_step.get(batch, 0)

    if "mixed" in sections:
        count, out_tokens, lengths = mixed_count, mixed_out, mixed_lengths
        requests = [[int(t) for t in rng.integers(0, vocab, size=n)] for n in lengths]
        for run in range(4):   # the first runs build kernels and meet every step shape and batch size (graphs are captured on the third use)
            steps_before = runner.steps
            torch.cuda.synchronize()
            started = time.perf_counter()
            results = engine.generate(requests, SamplingParams(max_tokens=out_tokens))
            torch.cuda.synchronize()
            seconds = time.perf_counter() - started
        points["mixed_requests"] = count
        points["mixed_prompt_tokens"] = sum(lengths)
        points["mixed_generated_tokens"] = sum(len(r.generated_tokens) for r in results)
        points["mixed_steps"] = runner.steps - steps_before
        points["mixed_preemptions"] = sum(r.preemptions for r in results)
        points["mixed_tokens_per_s"] = (sum(lengths) + points["mixed_generated_tokens"]) / seconds
        points["mixed_generated_per_s"] = points["mixed_generated_tokens"] / seconds

    return {
        "metric": metric_name(args, chosen),
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights N(0, 0.02), uniform random token ids)",
        "impl": "engine",
        "config": config_record(args, chosen, layers, first_context, peak_kind),
        "e2e": e2e,
        "gpu_launches": kernels_per_step * steps,
        "library_gemms_per_step": library_per_step.get(args.batch, 0),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s", "frac": achieved / peak["hbm_gbs"], "bytes_per_step": step_bytes},
        "points": points,
        "clocks": clocks,
    }


def run_reference(args) -> dict:
    """The unmodified reference on the same metric: TinyLlama 1.1B, 1,024-token prompts, greedy decoding, float16."""
    sys.path.insert(0, str(ROOT / "baseline"))
    import reference_arm

    try:
        if args.config != "tinyllama" or (args.layers or 22) != 22:
            raise reference_arm.Unavailable("the reference runs the TinyLlama-1.1B configuration with all 22 layers only (src/model_config.cpp:54-76)")
        chosen = CONFIGS["tinyllama"]
        if args.batch > 64:
            raise reference_arm.Unavailable("the reference's batched step takes at most 64 rows (src/cuda/model.cu:344-348)")
        warmup = max(args.warmup, 3)
        folder = model_folder("tinyllama", chosen["shapes"], 22)
        # the other batch sizes only on request: the reference feeds a prompt one position per step, three minutes for 64 requests
        batches = [args.batch] + [b for b in (1, 64) if b != args.batch and args.reference_points]
        with ClockSampler() as clocks:
            records = reference_arm.run(folder, chosen["prompt_tokens"], warmup, args.steps, batches)
    except reference_arm.Unavailable as reason:
        return {"impl": "reference", "unavailable": str(reason)}
    main_record = records[args.batch]
    peak, peak_kind = peaks()
    first_context = chosen["prompt_tokens"] + warmup
    step_bytes = decode_bytes(chosen["shapes"], 22, args.batch, first_context + (args.steps + 1) / 2.0)
    achieved = step_bytes / (main_record["device_ms_per_step"] / 1e3) / 1e9
    vocab = chosen["shapes"]["vocab_size"]
    return {
        "metric": metric_name(args, chosen),
        "value": args.batch * 1e3 / main_record["device_ms_per_step"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": main_record["device_ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16",
        "data": "synthetic (the engine arm's random weights as float16, uniform random token ids)", "impl": "reference",
        "config": config_record(args, chosen, 22, first_context, peak_kind),
        # a whole step of the reference's API: token ids in from the host, float16 logits of every row out and greedy on the host
        "e2e": {"value": args.batch * 1e3 / main_record["wall_ms_per_step"], "unit": "tokens/s", "h2d_bytes_per_step": args.batch * 4,
                "d2h_bytes_per_step": args.batch * vocab * 2},
        "gpu_launches": None, "prefill": None,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s", "frac": achieved / peak["hbm_gbs"], "bytes_per_step": step_bytes},
        "points": {f"decode_b{b}": b * 1e3 / records[b]["device_ms_per_step"] for b in records if b in (1, 64)},
        "clocks": clocks.summary(),
    }


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--config", default="tinyllama", choices=sorted(CONFIGS), help="whose layer sizes to run (random weights)")
    parser.add_argument("--layers", type=int, default=0, help="layers to run (default: all 22 of tinyllama, 8 of the 32 of the larger shapes)")
    parser.add_argument("--prefill-samples", type=int, default=5)
    parser.add_argument("--impl", default="engine", choices=["engine", "reference"])
    parser.add_argument("--reference-points", action="store_true", help="with --impl reference: also time batch 1 and 64 (minutes)")
    parser.add_argument("--sections", default="decode,e2e,prefill,points,mixed", help="which measurements to take (fewer for profiling runs; `mixed` adds requests of mixed length through the scheduler)")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: this engine is single-GPU by design (asked for {args.gpus})")
        return 2
    print(json.dumps(run_reference(args) if args.impl == "reference" else run_engine(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
