"""A plain, slow implementation of the Llama decoder: the tests' yardstick.

Whole sequences, no cache, no batching, one function for each part, 32-bit
arithmetic on the CPU, and no code shared with the engine.  Every function restates
a formula of the reference and cites where it stands there.  ``tests/golden``
holds logits that the reference's own compiled CPU model produced for a tiny random
checkpoint; ``test_plain.py`` compares this file with them.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np
import torch

_NP = {"F32": np.float32, "F16": np.float16, "I32": np.int32, "I64": np.int64}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """Minimal reader of its own (header length, JSON header, raw payload); values as float32."""
    raw = np.memmap(path, dtype=np.uint8, mode="r")
    (n,) = struct.unpack("<Q", raw[:8].tobytes())
    header = json.loads(raw[8 : 8 + n].tobytes())
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        begin, end = info["data_offsets"]
        blob = raw[8 + n + begin : 8 + n + end]
        if info["dtype"] == "BF16":
            value = torch.from_numpy(np.array(blob)).view(torch.bfloat16).to(torch.float32)   # exact: bfloat16 is the upper half of a float32
        else:
            value = torch.from_numpy(np.array(blob).view(_NP[info["dtype"]]).astype(np.float32))
        out[name] = value.reshape(info["shape"])
    return out


def load_model(folder) -> tuple[dict, dict[str, torch.Tensor]]:
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """src/operators.cpp:22-45: sum of squares in double, scale = 1/sqrt(float(mean) + eps), y = x*scale*w."""
    mean = (x.double() ** 2).sum(-1, keepdim=True) / x.shape[-1]
    scale = 1.0 / torch.sqrt(mean.float() + torch.tensor(eps, dtype=torch.float32))
    return x * scale * weight


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float, rotary_dim: int | None = None) -> torch.Tensor:
    """src/operators.cpp:47-78: pairs (d, d + D/2), frequency = pow(theta, -2d/D) in float, angle = pos * frequency.

    x: [tokens, heads, head_dim].
    """
    head_dim = x.shape[-1]
    rot = head_dim if rotary_dim is None else rotary_dim
    half = rot // 2
    d = torch.arange(half, dtype=torch.float32)
    frequency = torch.tensor(theta, dtype=torch.float32) ** (-2.0 * d / float(rot))
    angle = positions.to(torch.float32)[:, None] * frequency[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    first, second = x[..., :half], x[..., half:rot]
    out = x.clone()
    out[..., :half] = first * cos - second * sin
    out[..., half:rot] = second * cos + first * sin
    return out


def softmax_rows(scores: torch.Tensor) -> torch.Tensor:
    """src/operators.cpp:80-100: subtract the maximum, exp in float, sum in double, divide."""
    e = torch.exp(scores - scores.max(-1, keepdim=True).values)
    return (e.double() / e.double().sum(-1, keepdim=True)).float()


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0, scale: float | None = None) -> torch.Tensor:
    """src/operators.cpp:102-146 for every position of a sequence.

    q: [S, heads, D], k and v: [S, kv_heads, D].  Query i sees keys 0..i (the reference
    attends to the position+1 cached entries, src/model.cpp:159-169), or the last
    ``window`` of them.  kv head of query head h is h // (heads / kv_heads).
    """
    S, heads, D = q.shape
    groups = heads // k.shape[1]
    scale = (1.0 / np.sqrt(np.float32(D))) if scale is None else scale
    out = torch.zeros_like(q)
    # keys a query may not see get a score of -inf: exp gives exactly 0, so sums and products are those of the visible keys
    query, key = torch.arange(S)[:, None], torch.arange(S)[None, :]
    hidden = key > query
    if window > 0:
        hidden = hidden | (key < query - window + 1)
    for h in range(heads):
        g = h // groups
        scores = (q[:, h, :] @ k[:, g, :].T) * np.float32(scale)
        p = softmax_rows(scores.masked_fill(hidden, float("-inf")))
        out[:, h, :] = p @ v[:, g, :]
    return out


def silu_multiply(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """src/operators.cpp:148-164: (g / (1 + exp(-g))) * u."""
    return (gate / (1.0 + torch.exp(-gate))) * up


def linear(weight: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """src/model.cpp:53-78: y[o] = sum_i W[o, i] x[i], weights row-major [out, in]."""
    return x @ weight.T


def greedy(logits: torch.Tensor) -> int:
    """src/operators.cpp:166-175: the first maximum, i.e. the lowest id on ties."""
    return int(torch.nonzero(logits == logits.max())[0].item())


def forward(config: dict, w: dict[str, torch.Tensor], tokens: list[int], trace: dict | None = None, rows: list[int] | None = None) -> torch.Tensor:
    """Logits [len(tokens), vocab] of one whole sequence (src/model.cpp:80-234, one position at a time there).

    ``rows``: only these positions' logits (a large vocabulary makes the head the most expensive product of all).
    ``trace``: filled with every layer's output (the reference's ModelTrace, src/model.cpp:98-100, 200-206)."""
    H = config["hidden_size"]
    heads = config["num_attention_heads"]
    kv_heads = config.get("num_key_value_heads") or heads
    D = config.get("head_dim") or H // heads
    eps = config["rms_norm_eps"]
    theta = config.get("rope_theta", 10000.0)
    positions = torch.arange(len(tokens))
    hidden = w["model.embed_tokens.weight"][torch.tensor(tokens)]          # src/model.cpp:94-97
    for layer in range(config["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        normed = rms_norm(hidden, w[p + "input_layernorm.weight"], eps)   # :132
        q = linear(w[p + "self_attn.q_proj.weight"], normed).view(-1, heads, D)      # :140-146
        k = linear(w[p + "self_attn.k_proj.weight"], normed).view(-1, kv_heads, D)
        v = linear(w[p + "self_attn.v_proj.weight"], normed).view(-1, kv_heads, D)
        q, k = rope(q, positions, theta), rope(k, positions, theta)       # :150-151
        mixed = attention(q, k, v).reshape(len(tokens), heads * D)        # :167-169
        hidden = hidden + linear(w[p + "self_attn.o_proj.weight"], mixed)  # :171, 179
        normed = rms_norm(hidden, w[p + "post_attention_layernorm.weight"], eps)     # :180
        act = silu_multiply(linear(w[p + "mlp.gate_proj.weight"], normed), linear(w[p + "mlp.up_proj.weight"], normed))  # :187-195
        hidden = hidden + linear(w[p + "mlp.down_proj.weight"], act)      # :196-203
        if trace is not None:
            trace[f"layer{layer}.output"] = hidden.clone()
    if rows is not None:
        hidden = hidden[torch.tensor(rows, dtype=torch.long)]
    normed = rms_norm(hidden, w["model.norm.weight"], eps)                # :217
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return linear(head, normed)                                           # :225


def generate_greedy(config: dict, w: dict[str, torch.Tensor], prompt: list[int], max_tokens: int) -> list[int]:
    """app/reference_cli.cpp:89-110: feed the prompt, then max_tokens greedy tokens (no stop at EOS)."""
    tokens = list(prompt)
    out = []
    for _ in range(max_tokens):
        token = greedy(forward(config, w, tokens)[-1])
        out.append(token)
        tokens.append(token)
    return out


def sample_top_p(logits: torch.Tensor, temperature: float, top_p: float, uniform: float) -> int:
    """app/server.cpp:237-277 with the random number given: exp((l - max)/T), keep the most probable
    tokens until their share reaches top_p, draw in the kept mass.  The kept set is taken as
    {p >= p_of_the_token_that_crosses} (ties kept together) and walked in token-id order."""
    if not temperature > 0:
        return greedy(logits)
    p = torch.exp((logits - logits.max()) / np.float32(temperature)).float()
    total = float(p.double().sum())
    if top_p < 1.0:
        ordered = torch.sort(p, descending=True).values
        share = torch.cumsum(ordered.double(), 0) / total
        crossing = int(torch.nonzero(share >= top_p)[0].item())
        keep = p >= ordered[crossing]
    else:
        keep = torch.ones_like(p, dtype=torch.bool)
    kept = torch.where(keep, p, torch.zeros_like(p)).double()
    target = uniform * float(kept.sum())
    cursor = torch.cumsum(kept, 0)
    hits = torch.nonzero((cursor > target) & keep)
    return int(hits[0].item()) if len(hits) else int(torch.nonzero(keep)[-1].item())
