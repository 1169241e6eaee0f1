"""Generation through the entry point on the GPU: greedy ids, long decoding, first tokens, tight caches, graphs."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_llama
import tiny_configs
import trace_tools
from tinyllama_inference_engine_b200 import EngineConfig
from tinyllama_inference_engine_b200.engine.api import Engine
from tinyllama_inference_engine_b200.engine.request import SamplingParams
from tinyllama_inference_engine_b200.engine.runner import ModelRunner

pytestmark = pytest.mark.gpu


def _prompts(vocab, lengths, seed=1):
    rng = np.random.default_rng(seed)
    return [[int(t) for t in rng.integers(0, vocab, size=n)] for n in lengths]


def _engine(folder, **options):
    base = dict(dtype="float32", page_size=16, max_cache_tokens=1024, max_requests=8, max_batch_tokens=48)
    base.update(options)
    return Engine(folder, EngineConfig(**base))


def _agrees_up_to_near_ties(config, weights, prompt, got, want, fraction):
    """Equal ids, or at the first difference the chosen token's plain logit is within ``fraction`` of the scale of the top."""
    tokens = list(prompt)
    for a, b in zip(got, want):
        if a != b:
            logits = plain_llama.forward(config, weights, tokens)[-1]
            return float(logits.max() - logits[a]) <= fraction * float(logits.abs().max())
        tokens.append(a)
    return True


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("key", ["a", "b", "c"])
def test_greedy_generation_through_the_entry_point(model_folders, key, graphs):
    config, weights = plain_llama.load_model(model_folders[key])
    prompts = _prompts(config["vocab_size"], [1, 2, 7, 33])
    want = [plain_llama.generate_greedy(config, weights, p, 16) for p in prompts]
    engine = _engine(model_folders[key], use_cuda_graphs=graphs)
    got = [r.generated_tokens for r in engine.generate(prompts, SamplingParams(max_tokens=16))]
    assert got == want
    engine.runner.cache.check()
    bf16 = _engine(model_folders[key], dtype="bfloat16", use_cuda_graphs=graphs)
    got = [r.generated_tokens for r in bf16.generate(prompts, SamplingParams(max_tokens=16))]
    for prompt, g, w in zip(prompts, got, want):
        assert _agrees_up_to_near_ties(config, weights, prompt, g, w, 0.03)


def test_graph_and_eager_decoding_agree_and_sampling_is_seeded(model_folders):
    config, _ = plain_llama.load_model(model_folders["b"])
    prompts = _prompts(config["vocab_size"], [5, 40, 17, 64, 9], seed=4)
    params = [SamplingParams(max_tokens=20 + 7 * i, temperature=0.9, top_p=0.9, seed=i) for i in range(5)]
    eager = [r.generated_tokens for r in _engine(model_folders["b"], use_cuda_graphs=False).generate(prompts, params)]
    graph_engine = _engine(model_folders["b"], use_cuda_graphs=True)
    graphed = [r.generated_tokens for r in graph_engine.generate(prompts, params)]
    assert graphed == eager
    assert graph_engine._sessions, "decode steps should have gone through a graph session"
    alone = [_engine(model_folders["b"]).generate([p], [q])[0].generated_tokens for p, q in zip(prompts, params)]
    assert alone == eager  # a request's draws do not depend on the batch
    assert all(len(g) == p.max_tokens for g, p in zip(eager, params))


def test_long_decoding_stays_right(model_folders):
    """One token of prompt, then 250 decoded one by one: every step's logits against the plain implementation."""
    folder = model_folders["b"]
    config, weights = plain_llama.load_model(folder)
    requests = trace_tools.make_requests(config["vocab_size"], [251], seed=21)
    full = {rid: plain_llama.forward(config, weights, tokens) for rid, tokens in requests.items()}
    scale = max(float(v.abs().max()) for v in full.values())
    for dtype, fraction in (("float32", 2e-5), ("bfloat16", 2.5e-2)):
        runner = ModelRunner(folder, EngineConfig(dtype=dtype, page_size=16, max_cache_tokens=256, max_requests=2, max_batch_tokens=16))
        trace_tools.run_and_compare(runner, trace_tools.tail_decode(requests, tail=250), full, atol=fraction * scale)


def test_tight_cache_preempts_and_still_gives_the_same_tokens(model_folders):
    config, _ = plain_llama.load_model(model_folders["a"])
    prompts = _prompts(config["vocab_size"], [30, 30, 19, 25], seed=3)
    params = [SamplingParams(max_tokens=40, temperature=0.7, top_p=0.95, seed=50 + i) for i in range(4)]
    roomy = [r.generated_tokens for r in _engine(model_folders["a"]).generate(prompts, params)]
    tight_engine = _engine(model_folders["a"], max_cache_tokens=144)
    tight = [r.generated_tokens for r in tight_engine.generate(prompts, params)]
    assert tight_engine.metrics()["preemptions"] > 0 and tight == roomy
    tight_engine.runner.cache.check()
    assert tight_engine.runner.cache.free_pages() == tight_engine.runner.cache.total_pages()


def test_command_line_generates_on_the_gpu(model_folders, capsys):
    import json

    from tinyllama_inference_engine_b200.cli import main

    config, weights = plain_llama.load_model(model_folders["a"])
    prompt = _prompts(config["vocab_size"], [6], seed=2)[0]
    text = ",".join(map(str, prompt))
    assert main(["generate", str(model_folders["a"]), text, "8", "--dtype", "float32"]) == 0
    result = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    want = plain_llama.generate_greedy(config, weights, prompt, 8)
    assert result["generated_tokens"] == want and result["prompt_tokens"] == 6
    assert main(["reference", str(model_folders["a"]), text, "8", str(want[0]), "--dtype", "float32"]) == 0
    assert capsys.readouterr().out.splitlines()[0] == "token_ids:" + "".join(f" {t}" for t in want)
    assert main(["logits", str(model_folders["a"]), text, "--dtype", "float32"]) == 0
    logits = torch.tensor(json.loads(capsys.readouterr().out)["logits"])
    assert torch.allclose(logits, plain_llama.forward(config, weights, prompt)[-1], atol=1e-5)
    assert main(["benchmark", str(model_folders["a"]), "20", "6", "1", "2", "--batch", "2"]) == 0
    report = json.loads(capsys.readouterr().out)
    assert report["deterministic"] and report["median_decode_tokens_per_second"] > 0
    # the prompt as seeded random ids, the cache given in pages of 16, timings split as the reference splits them
    import numpy as np

    seeded = [int(t) for t in np.random.default_rng(5).integers(0, config["vocab_size"], size=9)]
    assert main(["generate", str(model_folders["a"]), "4", "--prompt-len", "9", "--prompt-seed", "5", "--page-size", "16", "--num-pages", "3", "--dtype", "float32"]) == 0
    result = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert result["generated_tokens"] == plain_llama.generate_greedy(config, weights, seeded, 4) and result["prompt_tokens"] == 9
    assert result["prefill_compute_ms"] > 0 and result["decode_compute_ms"] > 0 and result["decode_steps"] == 3
    assert result["prefill_transfer_ms"] >= 0 and result["decode_transfer_ms"] >= 0
    assert main(["generate", str(model_folders["a"]), "60", "--prompt-len", "9", "--page-size", "16", "--num-pages", "3"]) == 1   # 69 tokens do not fit three pages
    assert "error" in json.loads(capsys.readouterr().err.strip().splitlines()[-1])
    assert main(["generate", str(model_folders["a"]), text, "2", "--device", "cpu"]) == 1                                       # no CPU path, said loudly
    assert json.loads(capsys.readouterr().err.strip().splitlines()[-1])["error"]["code"] == "cuda"
    assert main(["kernel-bench", str(model_folders["b"]), "4", "100", "3"]) == 0
    kernels = json.loads(capsys.readouterr().out)["kernels"]
    assert {"add_rmsnorm", "rope_store", "linear_qkv", "attention_decode_split_kv", "argmax"} <= set(kernels)
    assert all(k["median_us"] > 0 for k in kernels.values())
    # a model of a config.json with seeded random weights, made on the spot: the same tokens as the folder written beforehand
    config_file = model_folders["a"] / "config.json"
    assert main(["generate", "-", text, "8", "--dtype", "float32", "--random-config", str(config_file), "--weights-seed", str(tiny_configs.ALL["a"][1])]) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["generated_tokens"] == want


def test_steps_launched_ahead_keep_the_engine_consistent(model_folders):
    """Pure decode steps are launched one ahead of their step() call; cancelling and adding requests meanwhile must not
    disturb anybody's tokens nor leak pages."""
    config, weights = plain_llama.load_model(model_folders["b"])
    prompts = _prompts(config["vocab_size"], [9, 30, 17, 5], seed=23)
    want = [plain_llama.generate_greedy(config, weights, p, 24) for p in prompts]
    engine = _engine(model_folders["b"], use_cuda_graphs=True)
    ids = [engine.add_request(p, SamplingParams(max_tokens=24)) for p in prompts[:3]]
    steps = 0
    late = None
    while engine.has_unfinished():
        engine.step()
        steps += 1
        if steps == 6:
            assert engine._ahead is not None, "a decode step should be in flight between step() calls"
            engine.cancel(ids[1])                                   # its token of the step in flight is dropped
            late = engine.add_request(prompts[3], SamplingParams(max_tokens=24))   # joins after the step in flight
        assert steps < 200
    assert engine.requests[ids[0]].generated == want[0]
    assert engine.requests[ids[2]].generated == want[2]
    assert engine.requests[late].generated == want[3]
    assert engine.requests[ids[1]].finish_reason == "cancelled" and len(engine.requests[ids[1]].generated) < 24
    assert engine.requests[ids[1]].generated == want[1][: len(engine.requests[ids[1]].generated)]
    engine.runner.cache.check()
    assert engine.runner.cache.free_pages() == engine.runner.cache.total_pages()


def test_batches_that_pass_through_a_size_are_not_captured(model_folders):
    """Requests finishing one per step: the sizes the batch only passes through run kernel by kernel, the lasting one as a graph."""
    config, weights = plain_llama.load_model(model_folders["b"])
    prompts = _prompts(config["vocab_size"], [9, 9, 9, 9], seed=8)
    params = [SamplingParams(max_tokens=n) for n in (12, 13, 14, 30)]
    engine = _engine(model_folders["b"], use_cuda_graphs=True)
    got = [r.generated_tokens for r in engine.generate(prompts, params)]
    assert got == [plain_llama.generate_greedy(config, weights, p, q.max_tokens) for p, q in zip(prompts, params)]
    sessions = engine._sessions
    assert sessions[4].graph is not None and sessions[1].graph is not None   # eleven and sixteen steps
    assert sessions[3].graph is None and sessions[2].graph is None           # one step each
    engine.runner.cache.check()


def test_one_token_prompts(model_folders):
    """A prompt of one token is a step of one token that samples, but of a request the cache does not know yet: it must not
    go the way of decode steps (which continue live requests), and what follows it must."""
    config, weights = plain_llama.load_model(model_folders["b"])
    prompts = [[7], [11], [3]]
    engine = _engine(model_folders["b"], use_cuda_graphs=True)
    got = [r.generated_tokens for r in engine.generate(prompts, SamplingParams(max_tokens=6))]
    assert got == [plain_llama.generate_greedy(config, weights, p, 6) for p in prompts]


@pytest.mark.parametrize("count", [12, 20])
def test_wider_decode_batches(model_folders, count):
    """Twelve requests decode on the 16-row fused kernels, twenty on the library's product with separate norm kernels."""
    config, weights = plain_llama.load_model(model_folders["e"])
    prompts = _prompts(config["vocab_size"], [3 + (5 * i) % 23 for i in range(count)], seed=12)
    want = [plain_llama.generate_greedy(config, weights, p, 10) for p in prompts]
    engine = _engine(model_folders["e"], dtype="bfloat16", use_cuda_graphs=True, max_requests=32, max_cache_tokens=4096, max_batch_tokens=256)
    got = [r.generated_tokens for r in engine.generate(prompts, SamplingParams(max_tokens=10))]
    for prompt, g, w in zip(prompts, got, want):
        assert _agrees_up_to_near_ties(config, weights, prompt, g, w, 0.03)
    assert count in engine._sessions
    engine.runner.cache.check()


def test_a_fault_recorded_on_the_device_fails_the_step(model_folders):
    """Kernels that give up a bounded wait, or meet a token id outside the vocabulary, set a bit in the device's error word.
    The engine reads the word where it waits for the device anyway, raises, and clears it; the failure is made on the host
    here (the word is written by the test), no kernel is driven into a fault."""
    from tinyllama_inference_engine_b200 import ops
    from tinyllama_inference_engine_b200.engine.replay import replay_step
    from tinyllama_inference_engine_b200.errors import KernelError

    engine = _engine(model_folders["a"], dtype="bfloat16", use_cuda_graphs=True)
    word = ops.error_flag(engine.runner.device)
    engine.add_request([5, 6, 7], SamplingParams(max_tokens=6))
    engine.step()                      # the prompt
    engine.step()                      # first decode steps, through a decode session
    word.fill_(1)
    with pytest.raises(KernelError, match="bounded wait"):
        for _ in range(3):
            engine.step()
    assert int(word.item()) == 0
    runner = ModelRunner(model_folders["a"], EngineConfig(dtype="float32", page_size=16, max_cache_tokens=64, max_requests=2, max_batch_tokens=16))
    word.fill_(2)
    with pytest.raises(KernelError, match="outside the vocabulary"):
        replay_step(runner, {"step": 0, "entries": [{"id": "x", "tokens": [1, 2], "want": [1]}], "end": ["x"]})
    assert replay_step(runner, {"step": 1, "entries": [{"id": "y", "tokens": [1, 2], "want": [1]}], "end": ["y"]}) is not None


def test_step_timings_and_layer_trace(model_folders):
    """A step that is asked says what it cost (device time of the forward pass and of the copies, host wall time), and can hand
    out the hidden state after every layer, which the plain implementation's trace locates a wrong layer with."""
    from tinyllama_inference_engine_b200.engine.batch import StepEntry
    from tinyllama_inference_engine_b200.engine.timing import StepTimings

    folder = model_folders["b"]
    config, weights = plain_llama.load_model(folder)
    tokens = _prompts(config["vocab_size"], [41], seed=4)[0]
    plain_trace: dict = {}
    plain = plain_llama.forward(config, weights, tokens, trace=plain_trace)
    for dtype, fraction in (("float32", 2e-5), ("bfloat16", 2.5e-2)):
        runner = ModelRunner(folder, EngineConfig(dtype=dtype, page_size=16, max_cache_tokens=64, max_requests=2, max_batch_tokens=64))
        timings, trace = StepTimings(), {}
        first = runner.step([StepEntry("r", tokens[:30], [29])], timings, trace)
        second_trace: dict = {}
        second = runner.step([StepEntry("r", tokens[30:], [10])], timings, second_trace)
        assert timings.steps == 2 and timings.compute_ms > 0 and timings.wall_ms >= timings.compute_ms * 0.5 and timings.transfer_ms >= 0
        assert float((first[0].cpu() - plain[29]).abs().max()) <= fraction * float(plain.abs().max())
        assert float((second[0].cpu() - plain[40]).abs().max()) <= fraction * float(plain.abs().max())
        assert set(trace) == {f"layer{i}.output" for i in range(config["num_hidden_layers"])}
        for name, want in plain_trace.items():
            got = torch.cat([trace[name], second_trace[name]]).cpu()
            assert got.shape == want.shape and float((got - want).abs().max()) <= fraction * float(want.abs().max()), name


@pytest.mark.parametrize("dtype,fraction", [("float32", 2e-5), ("bfloat16", 2.5e-2)])
def test_step_shapes_that_repeat_are_replayed_as_graphs(model_folders, dtype, fraction):
    """A step shape that comes up again is captured as a CUDA graph and replayed: other tokens, other positions, other pages
    and other wanted places each time, the same logits as the plain implementation every time."""
    from tinyllama_inference_engine_b200.engine.batch import StepEntry

    folder = model_folders["e"]
    config, weights = plain_llama.load_model(folder)
    runner = ModelRunner(folder, EngineConfig(dtype=dtype, page_size=64, max_cache_tokens=2048, max_requests=4, max_batch_tokens=512, use_cuda_graphs=True))
    prompts = _prompts(config["vocab_size"], [330, 330, 330, 330, 330], seed=31)
    worst = 0.0
    for index, tokens in enumerate(prompts):
        full = plain_llama.forward(config, weights, tokens)
        scale = float(full.abs().max())
        # the same three shapes for every request of 330 tokens: (150 tokens, 1 wanted), (150, 2), (30, 30); the pool hands out other pages
        cuts = [(0, 150, [149 - index]), (150, 300, [index, 149]), (300, len(tokens), list(range(len(tokens) - 300)))]
        for begin, end, want in cuts:
            got = runner.step([StepEntry(f"r{index}", tokens[begin:end], want)])
            expect = torch.stack([full[begin + w] for w in want])
            worst = max(worst, float((got.cpu() - expect).abs().max()) / scale)
        if index % 2:
            runner.finish(f"r{index}")   # some requests stay, so that later ones get other pages
    assert worst <= fraction, worst
    graphs = [slot for slot in runner._step_graphs.values() if slot.graph is not None]
    assert len(graphs) == 3 and all(slot.uses >= 4 for slot in graphs)
