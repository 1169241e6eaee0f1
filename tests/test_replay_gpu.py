"""The engine on the GPU, in 32-bit and in bfloat16, under every way of cutting the work, against the plain implementation."""
from __future__ import annotations

import pytest
import torch

import plain_llama
import trace_tools
from tinyllama_inference_engine_b200 import EngineConfig
from tinyllama_inference_engine_b200.engine.runner import ModelRunner

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("product_thresholds")]

# largest |difference| allowed, as a fraction of the largest |logit| of the request set
TOLERANCE = {"float32": 2e-5, "bfloat16": 2.5e-2}
LENGTHS = {"a": [1, 7, 33, 100, 128, 65], "b": [3, 19, 64, 100, 255, 130], "c": [2, 40, 77, 300, 129, 64], "d": [5, 200, 64, 1100, 129, 700],
           "e": [4, 640, 65, 31, 257, 128]}


@pytest.fixture(scope="module")
def cases(model_folders):
    out = {}
    for key, folder in model_folders.items():
        config, weights = plain_llama.load_model(folder)
        requests = trace_tools.make_requests(config["vocab_size"], LENGTHS[key], seed=11)
        full = {rid: plain_llama.forward(config, weights, tokens) for rid, tokens in requests.items()}
        scale = max(float(v.abs().max()) for v in full.values())
        out[key] = (folder, requests, full, scale)
    return out


def _runner(folder, dtype, max_tokens=2048, page_size=64):
    return ModelRunner(folder, EngineConfig(dtype=dtype, page_size=page_size, max_cache_tokens=max_tokens, max_requests=8, max_batch_tokens=2048, poison_freed_pages=True))


def test_far_key_decides_the_logits(model_folders):
    """Sharpened attention: with q and k projections scaled up, one early token dominates late positions, so a cache
    page misplaced or a key dropped far back changes the logits by much more than the tolerance."""
    import json

    from tinyllama_inference_engine_b200.weights import SafetensorsFile, write_safetensors

    source = model_folders["a"]
    folder = source.parent / "a_sharp"
    if not (folder / "model.safetensors").exists():
        folder.mkdir(exist_ok=True)
        (folder / "config.json").write_text((source / "config.json").read_text())
        file = SafetensorsFile(source / "model.safetensors")
        tensors = {name: file.tensor(name).clone() for name in file.names()}
        file.close()
        for name in tensors:
            if "q_proj" in name or "k_proj" in name:
                tensors[name] = (tensors[name].float() * 12.0).bfloat16()
        write_safetensors(folder / "model.safetensors", tensors)
    config, weights = plain_llama.load_model(folder)
    requests = trace_tools.make_requests(config["vocab_size"], [128, 100, 77], seed=17)
    full = {rid: plain_llama.forward(config, weights, tokens) for rid, tokens in requests.items()}
    scale = max(float(v.abs().max()) for v in full.values())
    for dtype in ("float32", "bfloat16"):
        for steps in (trace_tools.tail_decode(requests), trace_tools.portions(requests), trace_tools.mixed(requests, seed=9, page_size=16)[0]):
            runner = _runner(folder, dtype, max_tokens=1024, page_size=16)
            trace_tools.run_and_compare(runner, steps, full, atol=TOLERANCE[dtype] * scale)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_float16_checkpoint(tmp_path, dtype):
    """A checkpoint stored in float16 (the reference's GPU format, scripts/convert_model_fp16.py:23-67): the 32-bit engine sees
    every value exactly, so its logits meet the 32-bit bound; rounding the weights to bfloat16 first would miss it a hundredfold."""
    from tiny_configs import TINY_A
    from tinyllama_inference_engine_b200.weights import write_random_model

    folder = write_random_model(tmp_path / "half", TINY_A, seed=4, storage_dtype="float16")
    config, weights = plain_llama.load_model(folder)
    requests = trace_tools.make_requests(config["vocab_size"], [33, 100, 7], seed=12)
    full = {rid: plain_llama.forward(config, weights, tokens) for rid, tokens in requests.items()}
    scale = max(float(v.abs().max()) for v in full.values())
    for steps in (trace_tools.whole(requests), trace_tools.tail_decode(requests, tail=8)):
        trace_tools.run_and_compare(_runner(folder, dtype), steps, full, atol=TOLERANCE[dtype] * scale)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["a", "b", "c", "d", "e"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_replay(cases, key, dtype, cut):
    folder, requests, full, scale = cases[key]
    atol = TOLERANCE[dtype] * scale
    page_size = 16 if key == "c" else 64
    if cut == "mixed":
        steps, peak = trace_tools.mixed(requests, seed=5, page_size=page_size)
        runner = _runner(folder, dtype, max_tokens=peak, page_size=page_size)
    else:
        steps = {"whole": trace_tools.whole, "tail": trace_tools.tail_decode, "portions": trace_tools.portions}[cut](requests)
        runner = _runner(folder, dtype, page_size=page_size)
    worst = trace_tools.run_and_compare(runner, steps, full, atol=atol)
    runner.cache.check()
    assert not runner.cache.records
    if cut == "mixed":
        assert runner.cache.stats()["groups"][0]["reuses"] > 0
    print(f"{key} {dtype} {cut}: worst {worst:.3e} of scale {scale:.3f}")


@pytest.mark.parametrize("key", ["a", "b"])
def test_float32_rows_do_not_depend_on_the_cut(cases, key):
    """In 32-bit every kernel sums a row in an order of its own, so two cuts agree to the last bit."""
    folder, requests, full, scale = cases[key]
    from tinyllama_inference_engine_b200.engine.replay import replay_step

    rid = "r3"
    tokens = requests[rid]
    a = _runner(folder, "float32")
    whole = replay_step(a, {"step": 0, "entries": [{"id": rid, "tokens": tokens, "want": list(range(len(tokens)))}], "end": [rid]})
    b = _runner(folder, "float32")
    rows = []
    other = requests["r4"]
    for i, token in enumerate(tokens):
        entries = [{"id": rid, "tokens": [token], "want": [0]}]
        if i < len(other):
            entries.insert(0, {"id": "o", "tokens": [other[i]], "want": []})
        rows.append(replay_step(b, {"step": i, "entries": entries, "end": []})[0])
    assert torch.equal(torch.stack(rows), whole)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["d", "e"])
def test_mixed_steps_with_long_portions(cases, key, dtype):
    """Portions of up to 300 tokens that start anywhere inside a request, beside decoded tokens of up to three other requests:
    the tensor-core products, their accumulate epilogue and the prompt attention kernels (head size 128 and 64) in steps that also
    carry single rows, with a pool of exactly the peak so that pages are used again."""
    folder, requests, full, scale = cases[key]
    steps, peak = trace_tools.mixed(requests, seed=8, max_portion=300, page_size=64)
    assert max(len(e["tokens"]) for s in steps for e in s["entries"]) >= 128
    assert any(len(s["entries"]) > 1 and max(len(e["tokens"]) for e in s["entries"]) >= 128 and min(len(e["tokens"]) for e in s["entries"]) == 1 for s in steps)
    runner = _runner(folder, dtype, max_tokens=peak, page_size=64)
    worst = trace_tools.run_and_compare(runner, steps, full, atol=TOLERANCE[dtype] * scale)
    runner.cache.check()
    assert not runner.cache.records and runner.cache.stats()["groups"][0]["reuses"] > 0
    print(f"{key} {dtype} mixed with long portions: worst {worst:.3e} of scale {scale:.3f}")


def _crowd(folder, live: int, decoded: int, seed: int):
    """``live`` requests with prompts of mixed length, and the plain logits of each."""
    config, weights = plain_llama.load_model(folder)
    rng = __import__("numpy").random.default_rng(seed)
    lengths = [int(n) + decoded for n in rng.integers(3, 90, size=live)]
    requests = trace_tools.make_requests(config["vocab_size"], lengths, seed=seed + 1)
    full = {rid: plain_llama.forward(config, weights, tokens) for rid, tokens in requests.items()}
    return requests, full, max(float(v.abs().max()) for v in full.values())


@pytest.fixture
def skinny_products():
    """The engine's own tensor-core product for 17 to 127 rows (off by default: the library's product is ahead on the clock),
    with the fusions it brings: prepared norm in front, gate or residual add behind."""
    from tinyllama_inference_engine_b200.ops import fast

    fast.enable_skinny(True)
    yield
    fast.enable_skinny(False)


@pytest.mark.parametrize("key,live", [("e", 24), ("e", 64), ("d", 64), ("b", 33)])
def test_many_requests_decode_together_on_the_engines_own_products(model_folders, key, live, skinny_products):
    test_many_requests_decode_together(model_folders, key, live, "bfloat16")
    from tinyllama_inference_engine_b200.ops import fast

    assert fast.library_gemm_calls == test_many_requests_decode_together.library_calls_before   # nothing went to the library


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key,live", [("e", 24), ("e", 64), ("d", 64), ("b", 33)])
def test_many_requests_decode_together(model_folders, key, live, dtype):
    """24, 33 and 64 live requests: prompts in steps of several requests, then all of them decoding in one step, every row's logits
    compared.  Between 17 and 127 rows the bfloat16 products are not the small-step kernels any more, and with more (request, kv
    head) pairs than SMs decode attention runs its narrow build; neither is reached by four live requests."""
    decoded = 6
    folder = model_folders[key]
    requests, full, scale = _crowd(folder, live, decoded, seed=31)
    steps, ids = [], list(requests)
    for begin in range(0, live, 7):   # prompts, seven requests a step
        group = ids[begin : begin + 7]
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": requests[rid][:-decoded], "want": [len(requests[rid]) - decoded - 1]} for rid in group], "end": []})
    for k in range(decoded, 0, -1):   # then everybody decodes together
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [requests[rid][-k]], "want": [0]} for rid in ids], "end": ids if k == 1 else []})
    runner = ModelRunner(folder, EngineConfig(dtype=dtype, page_size=16 if key == "b" else 64, max_cache_tokens=live * 128, max_requests=live, max_batch_tokens=1024, poison_freed_pages=True))
    from tinyllama_inference_engine_b200.ops import fast

    test_many_requests_decode_together.library_calls_before = fast.library_gemm_calls
    # only the decode steps: prompts of several hundred rows may use the library's product for long K (ops.fast.tcgen05_takes)
    prompt_steps = [s for s in steps if len(s["entries"]) < live]
    worst = trace_tools.run_and_compare(runner, prompt_steps, full, atol=TOLERANCE[dtype] * scale)
    test_many_requests_decode_together.library_calls_before = fast.library_gemm_calls
    steps = [s for s in steps if len(s["entries"]) == live]
    runner.cache.check()
    print(f"{key} {live} live {dtype}: worst {worst:.3e} of scale {scale:.3f}")


@pytest.mark.parametrize("key,live", [("e", 64), ("d", 24)])
def test_decode_session_of_many_requests(model_folders, key, live):
    """The same crowd through a decode session: steps kernel by kernel, the capture, and replays of the graph, fed with given tokens;
    the logits of every step against the plain implementation."""
    from tinyllama_inference_engine_b200.engine.batch import StepEntry
    from tinyllama_inference_engine_b200.engine.decode_session import DecodeSession

    decoded = 6
    folder = model_folders[key]
    requests, full, scale = _crowd(folder, live, decoded, seed=37)
    ids = list(requests)
    runner = ModelRunner(folder, EngineConfig(dtype="bfloat16", page_size=64, max_cache_tokens=live * 128, max_requests=live, max_batch_tokens=1024))
    for rid in ids:
        runner.step([StepEntry(rid, requests[rid][:-decoded], [])])
    session = DecodeSession(runner, live)
    session.load(ids, [requests[rid][-decoded] for rid in ids])
    for k in range(decoded, 0, -1):
        if k != decoded:
            session.set_tokens([requests[rid][-k] for rid in ids])
        session.step()
        torch.cuda.synchronize()
        got = session.logits.float().cpu()
        want = torch.stack([full[rid][len(requests[rid]) - k] for rid in ids])
        error = float((got - want).abs().max())
        assert error <= TOLERANCE["bfloat16"] * scale, (k, error, scale)
    assert session.graph is not None   # the later steps were replays
