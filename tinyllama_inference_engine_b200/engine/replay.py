"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and owns no forward pass, cache or loader: every step goes through
``ModelRunner.step``, the step function generation uses.  The nearest things in the
reference are ``tinyllama_cuda logits`` (last-position logits as JSON,
app/cuda_reference.cu:228-254) and the traced CPU forward (src/model.cpp:98-100).

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
Output: ``<out>/<step>.f32`` (little-endian float32 [wanted, vocab]) for steps that
want something, and a flushed line ``done <step>`` after every step.  With
``--dump-layers`` also ``<out>/<step>.layers.f32``: the hidden state of every row of the
step after every run of a layer, float32 [layer runs, rows, hidden], for finding the
layer at which a wrong logit starts.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

from .. import ops
from ..config import EngineConfig
from ..errors import EngineError
from .batch import StepEntry

REPLAY_LIVE_REQUESTS = 8


def replay_engine_config(dtype: str, max_tokens: int, page_size: int = 64, device: str = "cuda:0") -> EngineConfig:
    """The engine options of a replay: a pool of exactly ``max_tokens`` (rounded up to whole pages)."""
    pages = max(1, -(-max_tokens // page_size))
    # a step can bring at most what the pool holds, so that is the step's token budget too
    return EngineConfig(dtype=dtype, page_size=page_size, max_cache_tokens=pages * page_size,
                        max_requests=REPLAY_LIVE_REQUESTS, max_batch_tokens=max(256, pages * page_size), device=device, use_cuda_graphs=False)


def replay_step(runner, step: dict, trace: dict | None = None):
    """Run one step of a trace; returns the wanted logits on the host (or None).  ``trace``: see ``ModelRunner.step``."""
    entries = [StepEntry(e["id"], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]) for e in step["entries"]]
    logits = runner.step(entries, trace=trace) if entries else None
    for request_id in step.get("end", []):
        runner.finish(request_id)
    if logits is None:
        return None
    host = logits.float().cpu()
    ops.check_device_errors(runner.device)   # a fault a kernel recorded on the device makes the step fail, not its logits wrong
    return host


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description="replay token ids through the engine and write logits")
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True, help="most tokens live requests hold at any time")
    parser.add_argument("--dump-layers", action="store_true", help="also write every step's hidden state after every layer (<step>.layers.f32)")
    args = parser.parse_args(argv)
    try:
        from .runner import ModelRunner

        out = Path(args.out)
        out.mkdir(parents=True, exist_ok=True)
        runner = ModelRunner(args.model, replay_engine_config(args.dtype, args.max_tokens))
        for line in sys.stdin:
            line = line.strip()
            if not line:
                continue
            step = json.loads(line)
            trace = {} if args.dump_layers else None
            logits = replay_step(runner, step, trace)
            if logits is not None:
                (out / f"{step['step']}.f32").write_bytes(logits.contiguous().numpy().astype("<f4").tobytes())
            if trace:
                import torch

                layers = torch.stack([trace[f"layer{i}.output"] for i in range(len(trace))]).cpu()
                (out / f"{step['step']}.layers.f32").write_bytes(layers.contiguous().numpy().astype("<f4").tobytes())
            print(f"done {step['step']}", flush=True)
        return 0
    except EngineError as exc:
        print(json.dumps(exc.to_json()), file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
