"""The plain implementation against the reference's own compiled CPU model, and against itself."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

import plain_llama
from tiny_configs import ALL

GOLDEN = json.loads((Path(__file__).parent / "golden" / "reference_logits.json").read_text())


def test_plain_matches_reference_binary(model_folders):
    """tests/golden/make_golden.py ran TinyLlamaCpu::Forward of the reference on these checkpoints."""
    for key in ("a", "b"):
        config, weights = plain_llama.load_model(model_folders[key])
        assert config["hidden_size"] == GOLDEN[key]["config"]["hidden_size"]
        logits = plain_llama.forward(config, weights, GOLDEN[key]["tokens"])
        want = torch.tensor(GOLDEN[key]["logits"], dtype=torch.float32)
        assert logits.shape == want.shape
        assert torch.allclose(logits, want, atol=2e-6, rtol=1e-5), float((logits - want).abs().max())
        assert torch.equal(logits.argmax(-1), want.argmax(-1))


def test_plain_prefix_property(model_folders):
    """Logits at a position depend only on the tokens up to it."""
    config, weights = plain_llama.load_model(model_folders["c"])
    tokens = [int(t) for t in np.random.default_rng(0).integers(0, config["vocab_size"], size=12)]
    whole = plain_llama.forward(config, weights, tokens)
    part = plain_llama.forward(config, weights, tokens[:7])
    assert torch.allclose(whole[:7], part, atol=1e-6)


def test_plain_operators():
    x = torch.tensor([[1.0, -2.0, 3.0, 0.5]])
    w = torch.tensor([1.0, 0.5, 2.0, 1.0])
    scale = 1.0 / np.sqrt((1 + 4 + 9 + 0.25) / 4 + 1e-5)
    assert torch.allclose(plain_llama.rms_norm(x, w, 1e-5), x * scale * w, atol=1e-6)
    # rotation by position 0 is the identity; rotation keeps the norm of every pair
    q = torch.randn(3, 2, 8)
    assert torch.equal(plain_llama.rope(q, torch.zeros(3, dtype=torch.long), 10000.0), q)
    r = plain_llama.rope(q, torch.tensor([1, 7, 4095]), 10000.0)
    assert torch.allclose((r[..., :4] ** 2 + r[..., 4:] ** 2), (q[..., :4] ** 2 + q[..., 4:] ** 2), atol=1e-5)
    p = plain_llama.softmax_rows(torch.tensor([[1000.0, 1000.0, -1000.0]]))
    assert torch.allclose(p, torch.tensor([[0.5, 0.5, 0.0]]))
    assert plain_llama.greedy(torch.tensor([0.1, 0.7, 0.7, 0.2])) == 1
    g, u = torch.tensor([0.0, 1.0]), torch.tensor([2.0, 3.0])
    assert torch.allclose(plain_llama.silu_multiply(g, u), torch.tensor([0.0, 3.0 / (1 + np.exp(-1.0))]).float(), atol=1e-6)


def test_plain_attention_window_and_groups():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    full = plain_llama.attention(q, k, v)
    assert torch.allclose(full[0, 0], v[0, 0], atol=1e-6)  # the first position sees only itself
    assert torch.allclose(full[0, 3], v[0, 1], atol=1e-6)  # query head 3 reads kv head 1
    windowed = plain_llama.attention(q, k, v, window=2)
    assert torch.allclose(windowed[:2], full[:2], atol=1e-6)
    assert not torch.allclose(windowed[5], full[5], atol=1e-4)


def test_plain_sampling():
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0])
    assert plain_llama.sample_top_p(logits, 0.0, 1.0, 0.3) == 0
    p = torch.softmax(logits, 0)
    assert plain_llama.sample_top_p(logits, 1.0, 1.0, float(p[0]) - 1e-3) == 0
    assert plain_llama.sample_top_p(logits, 1.0, 1.0, float(p[0]) + 1e-3) == 1
    assert plain_llama.sample_top_p(logits, 1.0, 0.5, 0.999) == 0      # only the top token is kept
    assert plain_llama.sample_top_p(logits, 1.0, 0.7, 0.999) == 1      # two tokens are kept
