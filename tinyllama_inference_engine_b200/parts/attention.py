"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import torch

from .. import ops
from .base import CacheNeed, LayerCache, Mixer, build_part, register_part
from .spec import PartSpec, TensorSpec


class Attention(Mixer):
    """q, k, v projections, position encoding, cache write, attention, output projection.

    params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``,
    ``position`` (a PartSpec), optional ``window`` (0 = every earlier token) and
    ``scale`` (default head_dim ** -0.5).
    tensors: ``<prefix>.{q,k,v}_proj.weight [heads * head_dim, hidden]``,
    ``<prefix>.o_proj.weight [hidden, num_heads * head_dim]``; no biases
    (src/model_config.cpp:81-95).

    The reference issues three projections (src/cuda/model.cu:412-421); here their
    weights are stacked once at load time and one product yields ``[q | k | v]``.
    """

    capturable = True
    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, d = spec["hidden_size"], spec["head_dim"]
        q, kv = spec["num_heads"] * d, spec["num_kv_heads"] * d
        return [
            TensorSpec(f"{prefix}.q_proj.weight", (q, hidden)),
            TensorSpec(f"{prefix}.k_proj.weight", (kv, hidden)),
            TensorSpec(f"{prefix}.v_proj.weight", (kv, hidden)),
            TensorSpec(f"{prefix}.o_proj.weight", (hidden, q)),
        ]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        return CacheNeed("pages", kv_heads=spec["num_kv_heads"], head_dim=spec["head_dim"], window=int(spec.get("window", 0) or 0))

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden = int(spec["hidden_size"])
        self.q_heads = int(spec["num_heads"])
        self.kv_heads = int(spec["num_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.window = int(spec.get("window", 0) or 0)
        scale = spec.get("scale")
        self.scale = float(scale) if scale is not None else self.head_dim ** -0.5
        dtype = runtime.dtype
        self.w_qkv = torch.cat([weights.get(f"{prefix}.{n}_proj.weight", dtype) for n in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = weights.get(f"{prefix}.o_proj.weight", dtype).contiguous()
        self.position = build_part("position", spec["position"], prefix, weights, runtime)
        self.qkv_width = (self.q_heads + 2 * self.kv_heads) * self.head_dim

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_o)

    def forward(self, x, ctx, cache: LayerCache, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        qkv = ws.get("qkv", tokens, self.qkv_width, dtype)
        if isinstance(x, ops.LazyNorm):
            ops.norm_linear(x, self.w_qkv, qkv)
        else:
            ops.linear(x, self.w_qkv, qkv)
        table = self.position.rotary_table()
        if table is None:
            self.position.apply(qkv, ctx, self.q_heads, self.kv_heads, self.head_dim)
            inv_freq, rotary_dim = None, 0
        else:
            inv_freq, rotary_dim = table
        mixed = ws.get("attention", tokens, self.q_heads * self.head_dim, dtype)
        ops.attention_step(qkv, ctx.positions, ctx.token_seq, cache.block_table, inv_freq, rotary_dim, cache.pages, mixed,
                           self.q_heads, self.kv_heads, self.head_dim, cache.page_size, self.window, self.scale,
                           write_cache=cache.writes, batch=ctx)
        if accumulate_into is not None:
            ops.linear_accumulate(mixed, self.w_o, accumulate_into, prepare)
            return None
        out = ws.get("mixer_out", tokens, self.hidden, dtype)
        ops.linear(mixed, self.w_o, out)
        return out


register_part("mixer", "attention", Attention)
