"""bin/trace_run as a user runs it: a child process fed one JSON line at a time, answering `done <step>` after each,
writing <step>.f32 only for steps that want something, exiting 0 when its input ends."""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_llama
import trace_tools

pytestmark = pytest.mark.gpu

PROGRAM = Path(__file__).resolve().parent.parent / "bin" / "trace_run"


@pytest.mark.parametrize("dtype,fraction", [("float32", 2e-5), ("bfloat16", 2.5e-2)])
def test_trace_run_answers_step_by_step(model_folders, tmp_path, dtype, fraction):
    folder = model_folders["b"]
    config, weights = plain_llama.load_model(folder)
    requests = trace_tools.make_requests(config["vocab_size"], [40, 3, 70, 33, 2, 65], seed=5)
    full = {rid: plain_llama.forward(config, weights, tokens) for rid, tokens in requests.items()}
    scale = max(float(v.abs().max()) for v in full.values())
    steps, peak = trace_tools.mixed(requests, seed=3, tail=8, max_portion=24, page_size=64)
    expected = trace_tools.expected_rows(steps, full)
    out = tmp_path / "out"
    env = dict(os.environ, PYTHONUNBUFFERED="1")
    child = subprocess.Popen([sys.executable, str(PROGRAM), "--model", str(folder), "--dtype", dtype, "--out", str(out), "--max-tokens", str(peak)],
                             stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for step in steps:
            child.stdin.write(json.dumps(step) + "\n")
            child.stdin.flush()
            line = child.stdout.readline().strip()
            while line and not line.startswith("done"):     # progress lines of a first compilation may come before
                line = child.stdout.readline().strip()
            assert line == f"done {step['step']}"
            path = out / f"{step['step']}.f32"
            if step["step"] in expected:
                want = expected[step["step"]]
                got = np.fromfile(path, dtype="<f4").reshape(want.shape)
                assert float(np.abs(got - want.numpy()).max()) <= fraction * scale
            else:
                assert not path.exists()
        child.stdin.close()
        assert child.wait(timeout=60) == 0
    finally:
        if child.poll() is None:
            child.kill()


def test_trace_run_reports_errors_as_json_and_fails(model_folders, tmp_path):
    """A step that breaks the rules (more tokens than --max-tokens holds) ends the program with a message, not a hang."""
    folder = model_folders["a"]
    child = subprocess.run([sys.executable, str(PROGRAM), "--model", str(folder), "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"],
                           input=json.dumps({"step": 0, "entries": [{"id": "x", "tokens": list(range(1, 100)), "want": [0]}], "end": []}) + "\n",
                           capture_output=True, text=True, timeout=300)
    assert child.returncode != 0
    assert "error" in (child.stdout + child.stderr).lower()


def test_trace_run_dumps_layers(model_folders, tmp_path):
    """--dump-layers: the hidden state after every layer, for every row of the step, beside the logits."""
    folder = model_folders["a"]
    config, weights = plain_llama.load_model(folder)
    tokens = trace_tools.make_requests(config["vocab_size"], [13], seed=2)["r0"]
    plain_trace: dict = {}
    plain_llama.forward(config, weights, tokens, trace=plain_trace)
    out = tmp_path / "o"
    step = {"step": 0, "entries": [{"id": "x", "tokens": tokens, "want": [12]}], "end": ["x"]}
    child = subprocess.run([sys.executable, str(PROGRAM), "--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-tokens", "64", "--dump-layers"],
                           input=json.dumps(step) + "\n", capture_output=True, text=True, timeout=300)
    assert child.returncode == 0 and "done 0" in child.stdout
    layers = np.fromfile(out / "0.layers.f32", dtype="<f4").reshape(config["num_hidden_layers"], 13, config["hidden_size"])
    for index in range(config["num_hidden_layers"]):
        want = plain_trace[f"layer{index}.output"].numpy()
        assert float(np.abs(layers[index] - want).max()) <= 2e-5 * float(np.abs(want).max())
