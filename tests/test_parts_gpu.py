"""Each part alone, built from a spec of its own (sizes unlike the model configurations') and random weights, against the
plain functions of tests/plain_llama.py: norm, position encoding, attention over a paged cache (two steps of one
request, with and without a window), gated feed-forward, the block that arranges them, embedding and head."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_llama
from tinyllama_inference_engine_b200.engine.batch import StepEntry, pack_step
from tinyllama_inference_engine_b200.parts import LayerCache, PartSpec, Runtime, Workspace, build_part
from tinyllama_inference_engine_b200.weights import WeightStore

pytestmark = pytest.mark.gpu

HIDDEN, HEADS, KV_HEADS, HEAD_DIM, INTER, PAGE = 136, 6, 3, 32, 200, 16
PRECISIONS = [(torch.float32, 3e-5), (torch.bfloat16, 2.5e-2)]


def _runtime(dtype):
    device = torch.device("cuda")
    return Runtime(dtype, device, Workspace(device, 64), {})


def _weights(named: dict[str, torch.Tensor]) -> WeightStore:
    """Random tensors that bfloat16 holds exactly, so both precisions see the same numbers."""
    return WeightStore({name: t.bfloat16().cuda() for name, t in named.items()}, "cuda")


def _close(got, want, fraction):
    want = want.float()
    assert float((got.float().cpu() - want).abs().max()) <= fraction * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype,fraction", PRECISIONS)
def test_rmsnorm_part(dtype, fraction):
    torch.manual_seed(0)
    weight = 1 + 0.2 * torch.randn(HIDDEN)
    part = build_part("norm", PartSpec("rmsnorm", {"size": HIDDEN, "eps": 3e-4}), "n", _weights({"n.weight": weight}), _runtime(dtype))
    residual, delta = torch.randn(7, HIDDEN) * 3, torch.randn(7, HIDDEN).bfloat16().float()
    got_residual = residual.clone().cuda()
    normed = part.forward(got_residual, delta.cuda().to(dtype))
    want = plain_llama.rms_norm(residual + delta, weight.bfloat16().float(), 3e-4)
    assert torch.allclose(got_residual.cpu(), residual + delta, atol=1e-6)     # the sum stays 32-bit
    _close(normed, want, fraction)
    rows = torch.tensor([5, 0, 2], dtype=torch.int32)
    some = part.forward(got_residual, None, rows=rows.cuda())
    _close(some, want[rows.long()], fraction)


def test_rotary_part_uses_the_plain_frequencies():
    part = build_part("position", PartSpec("rotary", {"rotary_dim": HEAD_DIM, "theta": 1234.5}), "p", _weights({}), _runtime(torch.float32))
    inv_freq, rotary_dim = part.rotary_table()
    exponent = (np.float32(-2.0) * np.arange(HEAD_DIM // 2, dtype=np.float32)) / np.float32(HEAD_DIM)
    assert rotary_dim == HEAD_DIM and np.array_equal(inv_freq.cpu().numpy(), np.power(np.float32(1234.5), exponent, dtype=np.float32))


def _attention_case(window):
    torch.manual_seed(3)
    spec = PartSpec("attention", {"hidden_size": HIDDEN, "num_heads": HEADS, "num_kv_heads": KV_HEADS, "head_dim": HEAD_DIM, "window": window,
                                  "scale": None, "position": PartSpec("rotary", {"rotary_dim": HEAD_DIM, "theta": 777.0})})
    named = {"a.q_proj.weight": torch.randn(HEADS * HEAD_DIM, HIDDEN) * 0.1, "a.k_proj.weight": torch.randn(KV_HEADS * HEAD_DIM, HIDDEN) * 0.1,
             "a.v_proj.weight": torch.randn(KV_HEADS * HEAD_DIM, HIDDEN) * 0.1, "a.o_proj.weight": torch.randn(HIDDEN, HEADS * HEAD_DIM) * 0.1}
    return spec, {k: v.bfloat16().float() for k, v in named.items()}


def _plain_attention(w, x, window):
    tokens = x.shape[0]
    positions = torch.arange(tokens)
    q = plain_llama.linear(w["a.q_proj.weight"], x).view(tokens, HEADS, HEAD_DIM)
    k = plain_llama.linear(w["a.k_proj.weight"], x).view(tokens, KV_HEADS, HEAD_DIM)
    v = plain_llama.linear(w["a.v_proj.weight"], x).view(tokens, KV_HEADS, HEAD_DIM)
    q, k = plain_llama.rope(q, positions, 777.0), plain_llama.rope(k, positions, 777.0)
    mixed = plain_llama.attention(q, k, v, window=window)
    return plain_llama.linear(w["a.o_proj.weight"], mixed.reshape(tokens, HEADS * HEAD_DIM))


@pytest.mark.parametrize("window", [0, 5])
@pytest.mark.parametrize("dtype,fraction", PRECISIONS)
def test_attention_part_over_a_paged_cache(dtype, fraction, window):
    """37 tokens of one request in a step of 30 and a step of 7 (cut inside a page), pages in scrambled order."""
    spec, named = _attention_case(window)
    runtime = _runtime(dtype)
    part = build_part("mixer", spec, "a", _weights(named), runtime)
    need = part.cache_need(spec)
    assert (need.kind, need.kv_heads, need.head_dim, need.window) == ("pages", KV_HEADS, HEAD_DIM, window)
    x = torch.randn(37, HIDDEN).bfloat16().float()
    want = _plain_attention(named, x, window)
    pages = torch.full((8, 2, KV_HEADS, PAGE, HEAD_DIM), float("nan"), dtype=dtype, device="cuda")
    row = [6, 1, 4]                                  # the request's pages, not in order
    got = []
    for first, count in ((0, 30), (30, 7)):
        table_rows = [[row + [-1]]]
        ctx = pack_step([StepEntry("r", [0] * count, [])], [first], [0], table_rows, runtime.device)
        cache = LayerCache(need, True, pages, ctx.block_tables[0], PAGE, None)
        out = part.forward(x[first : first + count].cuda().to(dtype), ctx, cache)
        got.append(out.float().cpu().clone())
    _close(torch.cat(got), want, fraction)
    assert not torch.isnan(pages[row, :, :, :, :].view(3, 2, KV_HEADS, PAGE, HEAD_DIM)[:2]).any()   # two full pages were written
    assert torch.isnan(pages[0]).all()                                                          # and no page it does not hold


@pytest.mark.parametrize("dtype,fraction", PRECISIONS)
def test_gated_feed_forward_part(dtype, fraction):
    torch.manual_seed(5)
    named = {"m.gate_proj.weight": torch.randn(INTER, HIDDEN) * 0.1, "m.up_proj.weight": torch.randn(INTER, HIDDEN) * 0.1,
             "m.down_proj.weight": torch.randn(HIDDEN, INTER) * 0.1}
    named = {k: v.bfloat16().float() for k, v in named.items()}
    runtime = _runtime(dtype)
    part = build_part("feed_forward", PartSpec("gated_mlp", {"hidden_size": HIDDEN, "intermediate_size": INTER, "activation": "silu"}), "m", _weights(named), runtime)
    for tokens in (3, 40):                            # the few-row kernels and the many-row ones
        x = torch.randn(tokens, HIDDEN).bfloat16().float()
        want = plain_llama.linear(named["m.down_proj.weight"], plain_llama.silu_multiply(plain_llama.linear(named["m.gate_proj.weight"], x), plain_llama.linear(named["m.up_proj.weight"], x)))
        got = part.forward(x.cuda().to(dtype), None)
        _close(got, want, fraction)


@pytest.mark.parametrize("tokens", [5, 40])
@pytest.mark.parametrize("dtype,fraction", PRECISIONS)
def test_block_part_arranges_norms_mixer_and_feed_forward(dtype, fraction, tokens):
    """residual' = r + attention(norm(r)); out = residual' + mlp(norm(residual')), for few rows (fused kernels) and many."""
    torch.manual_seed(7)
    attention_spec, named = _attention_case(0)
    norm = PartSpec("rmsnorm", {"size": HIDDEN, "eps": 1e-5})
    mlp = PartSpec("gated_mlp", {"hidden_size": HIDDEN, "intermediate_size": INTER, "activation": "silu"})
    spec = PartSpec("pre_norm_residual", {"mixer_norm": norm, "mixer_norm_name": "n1", "mixer": attention_spec, "mixer_name": "att",
                                          "feed_forward_norm": norm, "feed_forward_norm_name": "n2", "feed_forward": mlp, "feed_forward_name": "ff"})
    named = {"b.att." + k[2:]: v for k, v in named.items()}
    named.update({"b.n1.weight": 1 + 0.1 * torch.randn(HIDDEN), "b.n2.weight": 1 + 0.1 * torch.randn(HIDDEN), "b.ff.gate_proj.weight": torch.randn(INTER, HIDDEN) * 0.1,
                  "b.ff.up_proj.weight": torch.randn(INTER, HIDDEN) * 0.1, "b.ff.down_proj.weight": torch.randn(HIDDEN, INTER) * 0.1})
    named = {k: v.bfloat16().float() for k, v in named.items()}
    runtime = _runtime(dtype)
    block = build_part("block", spec, "b", _weights(named), runtime)
    residual = torch.randn(tokens, HIDDEN).bfloat16().float()
    plain_w = {"a." + k[6:]: v for k, v in named.items() if k.startswith("b.att.")}
    middle = residual + _plain_attention(plain_w, plain_llama.rms_norm(residual, named["b.n1.weight"], 1e-5), 0)
    x = plain_llama.rms_norm(middle, named["b.n2.weight"], 1e-5)
    want = middle + plain_llama.linear(named["b.ff.down_proj.weight"], plain_llama.silu_multiply(plain_llama.linear(named["b.ff.gate_proj.weight"], x), plain_llama.linear(named["b.ff.up_proj.weight"], x)))
    pages = torch.zeros((4, 2, KV_HEADS, PAGE, HEAD_DIM), dtype=dtype, device="cuda")
    ctx = pack_step([StepEntry("r", [0] * tokens, [])], [0], [0], [[[2, 0, 3, -1]]], runtime.device)
    cache = LayerCache(block.cache_need(spec), True, pages, ctx.block_tables[0], PAGE, None)
    got_residual, delta = block.forward(residual.clone().cuda(), None, ctx, cache)
    got = got_residual.float().cpu() if delta is None else got_residual.float().cpu() + delta.float().cpu()
    _close(got, want, fraction)


@pytest.mark.parametrize("dtype,fraction", PRECISIONS)
def test_embedding_and_head_parts(dtype, fraction):
    torch.manual_seed(9)
    vocab = 131
    table = torch.randn(vocab, HIDDEN).bfloat16().float()
    own = (torch.randn(vocab, HIDDEN) * 0.1).bfloat16().float()
    runtime = _runtime(dtype)
    weights = _weights({"emb.weight": table, "out.weight": own})
    embedding = build_part("embedding", PartSpec("token_embedding", {"vocab_size": vocab, "hidden_size": HIDDEN, "name": "emb"}), "", weights, runtime)
    ids = torch.tensor([130, 0, 7, 7], dtype=torch.int32)
    residual = embedding.forward(ids.cuda())
    assert residual.dtype == torch.float32 and torch.equal(residual.cpu(), table[ids.long()])
    x = torch.randn(4, HIDDEN).bfloat16().float()
    # untied: its own tensor; tied without a tensor of its own: the embedding table; tied with one stored all the same: that one
    for tied, stored, matrix in ((None, weights, own), ("emb", _weights({"emb.weight": table}), table), ("emb", weights, own)):
        head = build_part("head", PartSpec("linear_head", {"vocab_size": vocab, "hidden_size": HIDDEN, "name": "out", "tied_to": tied}), "", stored, runtime)
        logits = head.forward(x.cuda().to(dtype))
        assert logits.dtype == torch.float32
        _close(logits, plain_llama.linear(matrix, x), fraction)
