"""The assembled model at the widths of real Llama checkpoints, against the plain implementation.

Two layers each of the TinyLlama-1.1B, Llama-2-7B and Llama-3-8B shapes (hidden, intermediate, heads, head size, vocabulary
and theta as those checkpoints have them) with random weights.  At these widths the engine chooses kernels and tile shapes
the tiny configurations never reach: the tcgen05 products with their wave-fitted tile widths, the SM-pair product and the
library rule for long K, the sixteen-warp down projection of decode steps, the tensor-memory attention at head size 64 and
128, a vocabulary of 128,256.  The reference's whole-model gate is tests/m1_integration_tests.cpp:92-152 and
scripts/compare_logits.py:101-172 (its own logits against a trusted forward at the real size).

Each shape: one prompt whole in one step, the same prompt in two portions (the second starts inside a page and carries
128 rows or more), and eight more tokens decoded one by one after each, in 32-bit and in bfloat16.
"""
from __future__ import annotations

import gc

import pytest
import torch

import plain_llama
import trace_tools
from tinyllama_inference_engine_b200 import EngineConfig
from tinyllama_inference_engine_b200.engine.runner import ModelRunner
from tinyllama_inference_engine_b200.weights import write_random_model

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("product_thresholds")]

TOLERANCE = {"float32": 2e-5, "bfloat16": 2.5e-2}   # of the largest |logit|, as everywhere in these tests

_COMMON = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=2, rms_norm_eps=1e-5, tie_word_embeddings=False,
               hidden_act="silu", attention_bias=False, bos_token_id=1, eos_token_id=2, torch_dtype="bfloat16")
SHAPES = {
    # name: (config, prompt tokens, where the prompt is cut in two)
    "tinyllama-1.1b": (dict(_COMMON, hidden_size=2048, intermediate_size=5632, num_attention_heads=32, num_key_value_heads=4,
                            max_position_embeddings=2048, vocab_size=32000, rope_theta=10000.0), 1100, 41),
    "llama2-7b": (dict(_COMMON, hidden_size=4096, intermediate_size=11008, num_attention_heads=32, num_key_value_heads=32,
                       max_position_embeddings=4096, vocab_size=32000, rope_theta=10000.0), 300, 150),
    "llama3-8b": (dict(_COMMON, hidden_size=4096, intermediate_size=14336, num_attention_heads=32, num_key_value_heads=8,
                       max_position_embeddings=8192, vocab_size=128256, rope_theta=500000.0), 300, 171),
}
DECODED = 8


def _steps(tokens: list[int], prompt: int, cut: int | None, wanted: list[int]) -> list[dict]:
    """The prompt in one step or in two, then the remaining tokens one by one; ``wanted``: prompt positions whose logits are compared."""
    steps = []
    bounds = [0, prompt] if cut is None else [0, cut, prompt]
    for begin, end in zip(bounds, bounds[1:]):
        steps.append({"step": len(steps), "entries": [{"id": "r", "tokens": tokens[begin:end], "want": [w - begin for w in wanted if begin <= w < end]}], "end": []})
    for i in range(prompt, len(tokens)):
        steps.append({"step": len(steps), "entries": [{"id": "r", "tokens": [tokens[i]], "want": [0]}], "end": ["r"] if i == len(tokens) - 1 else []})
    return steps


@pytest.fixture(scope="module", params=list(SHAPES))
def case(request, tmp_path_factory):
    config, prompt, cut = SHAPES[request.param]
    folder = write_random_model(tmp_path_factory.mktemp(request.param) / "model", config, seed=3)
    loaded, weights = plain_llama.load_model(folder)
    tokens = trace_tools.make_requests(config["vocab_size"], [prompt + DECODED], seed=23)["r0"]
    wanted = sorted({0, 63, 64, 127, 128, cut - 1, cut, prompt - 1})
    rows = wanted + list(range(prompt, prompt + DECODED))
    plain = plain_llama.forward(loaded, weights, tokens, rows=rows)
    del weights
    gc.collect()
    full = torch.full((len(tokens), config["vocab_size"]), float("nan"))
    full[torch.tensor(rows)] = plain
    yield folder, tokens, prompt, cut, wanted, {"r": full}, float(plain.abs().max())
    gc.collect()
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_widths_match_the_plain_implementation(case, dtype):
    folder, tokens, prompt, cut, wanted, full, scale = case
    for where in (None, cut):
        runner = ModelRunner(folder, EngineConfig(dtype=dtype, page_size=64, max_cache_tokens=2048, max_requests=2, max_batch_tokens=prompt))
        worst = trace_tools.run_and_compare(runner, _steps(tokens, prompt, where, wanted), full, atol=TOLERANCE[dtype] * scale)
        print(f"{folder.parent.name} {dtype} cut {where}: worst {worst:.3e} of scale {scale:.3f}")
        del runner
        gc.collect()
        torch.cuda.empty_cache()
