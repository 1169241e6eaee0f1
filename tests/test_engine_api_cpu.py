"""The Python entry point and the command line on the CPU, with the kernels replaced by their plain functions."""
from __future__ import annotations

import json

import numpy as np
import pytest

import plain_llama
import plain_ops
from tinyllama_inference_engine_b200 import EngineConfig
from tinyllama_inference_engine_b200.engine.api import Engine
from tinyllama_inference_engine_b200.engine.request import SamplingParams
from tinyllama_inference_engine_b200.errors import EngineError


def _engine(folder, **options):
    base = dict(dtype="float32", page_size=16, max_cache_tokens=512, max_requests=4, max_batch_tokens=32, device="cpu")
    base.update(options)
    return Engine(folder, EngineConfig(**base))


def _prompts(vocab, lengths, seed=1):
    rng = np.random.default_rng(seed)
    return [[int(t) for t in rng.integers(0, vocab, size=n)] for n in lengths]


def test_greedy_generation_matches_the_plain_implementation(model_folders, monkeypatch):
    plain_ops.install(monkeypatch)
    config, weights = plain_llama.load_model(model_folders["a"])
    prompts = _prompts(config["vocab_size"], [1, 7, 33])
    engine = _engine(model_folders["a"])
    results = engine.generate(prompts, SamplingParams(max_tokens=16))
    for prompt, result in zip(prompts, results):
        assert result.generated_tokens == plain_llama.generate_greedy(config, weights, prompt, 16)
        assert result.finish_reason == "length"
    engine.runner.cache.check()
    assert engine.metrics()["cache"]["live_requests"] == 0


def test_preemption_recomputes_and_gives_the_same_tokens(model_folders, monkeypatch):
    plain_ops.install(monkeypatch)
    config, _ = plain_llama.load_model(model_folders["b"])
    prompts = _prompts(config["vocab_size"], [30, 30, 19], seed=3)
    params = [SamplingParams(max_tokens=40, temperature=0.8, top_p=0.9, seed=4 + i) for i in range(3)]
    roomy = _engine(model_folders["b"], max_cache_tokens=1024).generate(prompts, params)
    tight_engine = _engine(model_folders["b"], max_cache_tokens=112)  # 7 pages: not enough for all three to finish side by side
    tight = tight_engine.generate(prompts, params)
    assert tight_engine.metrics()["preemptions"] > 0
    assert [r.generated_tokens for r in tight] == [r.generated_tokens for r in roomy]
    assert sum(r.preemptions for r in tight) == tight_engine.metrics()["preemptions"]
    tight_engine.runner.cache.check()


def test_sampling_does_not_depend_on_the_batch(model_folders, monkeypatch):
    plain_ops.install(monkeypatch)
    config, _ = plain_llama.load_model(model_folders["a"])
    prompts = _prompts(config["vocab_size"], [5, 9, 3], seed=7)
    params = [SamplingParams(max_tokens=12, temperature=1.0, top_p=0.95, seed=10 + i) for i in range(3)]
    together = _engine(model_folders["a"]).generate(prompts, params)
    alone = [_engine(model_folders["a"]).generate([p], [q])[0] for p, q in zip(prompts, params)]
    assert [r.generated_tokens for r in together] == [r.generated_tokens for r in alone]
    other_seed = _engine(model_folders["a"]).generate([prompts[0]], [SamplingParams(max_tokens=12, temperature=1.0, top_p=0.95, seed=99)])[0]
    assert other_seed.generated_tokens != alone[0].generated_tokens


def test_eos_stop_and_cancel_and_refusals(model_folders, monkeypatch):
    plain_ops.install(monkeypatch)
    config, weights = plain_llama.load_model(model_folders["a"])
    prompt = _prompts(config["vocab_size"], [6], seed=9)[0]
    greedy = plain_llama.generate_greedy(config, weights, prompt, 8)
    engine = _engine(model_folders["a"])
    engine.model_config = type("C", (), {"eos_token_id": greedy[3]})()
    stopped = engine.generate([prompt], SamplingParams(max_tokens=8, ignore_eos=False))[0]
    first_hit = greedy.index(greedy[3])
    assert stopped.generated_tokens == greedy[: first_hit + 1] and stopped.finish_reason == "stop"
    kept = engine.generate([prompt], SamplingParams(max_tokens=8))[0]  # the reference's behaviour: exactly max_tokens
    assert kept.generated_tokens == greedy
    rid = engine.add_request(prompt, SamplingParams(max_tokens=50))
    engine.step()
    engine.cancel(rid)
    assert not engine.has_unfinished() and engine.requests[rid].finish_reason == "cancelled"
    engine.runner.cache.check()
    assert engine.runner.cache.free_pages() == engine.runner.cache.total_pages()
    with pytest.raises(EngineError, match="outside the model vocabulary"):
        engine.add_request([999999])
    with pytest.raises(EngineError, match="context length"):
        engine.add_request([1] * 120, SamplingParams(max_tokens=20))
    with pytest.raises(EngineError, match="max_tokens"):
        SamplingParams(max_tokens=0)
    with pytest.raises(EngineError, match="top_p"):
        SamplingParams(top_p=0.0)


def test_command_line_errors_have_the_reference_shape(model_folders, capsys):
    from tinyllama_inference_engine_b200.cli import main

    assert main(["generate", str(model_folders["a"]), "1 2 3", "zero"]) == 1
    error = json.loads(capsys.readouterr().err.strip().splitlines()[-1])
    assert error["error"]["code"] == "invalid_argument" and "MAX_TOKENS" in error["error"]["message"]
    assert main(["logits", str(model_folders["a"])]) == 1
    assert json.loads(capsys.readouterr().err.strip().splitlines()[0])["error"]["code"] == "invalid_argument"
    assert main(["generate", str(model_folders["a"]), "hello world", "4"]) == 1
    assert json.loads(capsys.readouterr().err.strip().splitlines()[-1])["error"]["code"] == "tokenizer"


def test_command_line_writes_a_random_model(tmp_path, capsys):
    from tiny_configs import TINY_C
    from tinyllama_inference_engine_b200.cli import main

    (tmp_path / "c.json").write_text(json.dumps(TINY_C))
    assert main(["random-model", str(tmp_path / "out"), str(tmp_path / "c.json"), "5"]) == 0
    assert (tmp_path / "out" / "config.json").exists() and (tmp_path / "out" / "model.safetensors").exists()
