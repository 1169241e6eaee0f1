"""Plain restatements of what each kernel of the engine must compute.

One function per kernel, same arguments as the host wrapper in
``tinyllama_inference_engine_b200.ops``, written with ordinary tensor operations in
32-bit arithmetic, paged exactly as the kernels are.  They serve two purposes: the
``-m gpu`` tests compare every kernel with its function here, and the CPU tests put
them in the wrappers' place (``install``) to exercise the engine's host logic (cache
manager, batching, step function) on a machine without a GPU.  Nothing in the
product imports this file.
"""
from __future__ import annotations

import numpy as np
import torch


def _store(out: torch.Tensor, value: torch.Tensor) -> None:
    out.copy_(value.to(out.dtype))


def embedding(table, ids, residual) -> None:
    _store(residual, table[ids.long()].float())


def add_rmsnorm(residual, delta, weight, eps, out, rows=None) -> None:
    if delta is not None:
        residual += delta.float()
    x = residual if rows is None else residual[rows.long()]
    scale = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + np.float32(eps))
    _store(out, (x * scale) * weight)


def add_(residual, delta) -> None:
    residual += delta.float()


def silu_mul(gate_up, out) -> None:
    inter = out.shape[1]
    g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
    _store(out, (g / (1.0 + torch.exp(-g))) * u)


def linear(x, weight, out) -> None:
    _store(out, x.float() @ weight.float().T)


def fused_rows_limit(dtype, device) -> int:
    return 0


def rope_store(qkv, positions, token_seq, block_table, inv_freq, rotary_dim, pages, q_heads, kv_heads, head_dim, page_size, write_cache=True) -> None:
    tokens = qkv.shape[0]
    view = qkv.view(tokens, q_heads + 2 * kv_heads, head_dim)
    rotated = view[:, : q_heads + kv_heads].float().clone()
    if inv_freq is not None and rotary_dim > 0:
        half = rotary_dim // 2
        angle = positions.float()[:, None] * inv_freq[None, :]
        cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        first, second = rotated[..., :half].clone(), rotated[..., half:rotary_dim].clone()
        rotated[..., :half] = first * cos - second * sin
        rotated[..., half:rotary_dim] = second * cos + first * sin
    view[:, :q_heads] = rotated[:, :q_heads].to(qkv.dtype)
    if not write_cache:
        return
    k = rotated[:, q_heads:].to(qkv.dtype)
    v = view[:, q_heads + kv_heads :]
    for t in range(tokens):
        pos = int(positions[t])
        page = int(block_table[int(token_seq[t]), pos // page_size])
        assert page >= 0, "a token is written to a page its request does not hold"
        pages[page, 0, :, pos % page_size, :] = k[t]
        pages[page, 1, :, pos % page_size, :] = v[t]


def paged_attention(qkv, pages, positions, token_seq, block_table, out, q_heads, kv_heads, head_dim, page_size, window=0, scale=None, batch=None) -> None:
    tokens = qkv.shape[0]
    scale = head_dim ** -0.5 if scale is None else scale
    q = qkv.view(tokens, -1, head_dim)[:, :q_heads].float()
    group = q_heads // kv_heads
    result = torch.zeros(tokens, q_heads, head_dim)
    for t in range(tokens):
        pos = int(positions[t])
        lo = max(0, pos - window + 1) if window > 0 else 0
        keys = torch.arange(lo, pos + 1)
        page_ids = block_table[int(token_seq[t]), keys // page_size].long()
        assert bool((page_ids >= 0).all()), "attention reads a page its request does not hold"
        k = pages[page_ids, 0, :, keys % page_size, :].float()  # [keys, kv_heads, D]
        v = pages[page_ids, 1, :, keys % page_size, :].float()
        for h in range(q_heads):
            s = (k[:, h // group, :] @ q[t, h]) * np.float32(scale)
            p = torch.softmax(s, 0)
            result[t, h] = p @ v[:, h // group, :]
    _store(out, result.view(tokens, q_heads * head_dim))


def attention_step(qkv, positions, token_seq, block_table, inv_freq, rotary_dim, pages, out, q_heads, kv_heads, head_dim, page_size,
                   window=0, scale=None, write_cache=True, batch=None) -> None:
    rope_store(qkv, positions, token_seq, block_table, inv_freq, rotary_dim, pages, q_heads, kv_heads, head_dim, page_size, write_cache)
    paged_attention(qkv, pages, positions, token_seq, block_table, out, q_heads, kv_heads, head_dim, page_size, window, scale, batch)


def argmax(logits, out) -> None:
    for r in range(logits.shape[0]):
        out[r] = int(torch.nonzero(logits[r] == logits[r].max())[0])


def uniform_from(seed: int, counter: int) -> float:
    mask = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + (counter + 1) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return (z >> 40) / 16777216.0


def sample(logits, temperature, top_p, seeds, counters, out) -> None:
    import plain_llama

    for r in range(logits.shape[0]):
        u = uniform_from(int(seeds[r]), int(counters[r]))
        out[r] = plain_llama.sample_top_p(logits[r].float(), float(temperature[r]), float(top_p[r]), u)


def can_accumulate(rows: int, weight) -> bool:
    return False   # no product adds into the residual here: the block adds the part's output in the norm that follows


_NAMES = ["embedding", "add_rmsnorm", "add_", "silu_mul", "linear", "fused_rows_limit", "rope_store", "paged_attention", "attention_step", "argmax", "sample",
          "can_accumulate"]


def install(monkeypatch) -> None:
    """Put these functions in the place of the kernel wrappers (CPU tests of host logic only)."""
    from tinyllama_inference_engine_b200 import ops

    for name in _NAMES:
        monkeypatch.setattr(ops, name, globals()[name])
