"""A decoder assembled from a ModelSpec: embedding, the ordered runs of blocks, norm, head."""
from __future__ import annotations

from ..parts.base import CacheNeed, LayerCache, Runtime, build_part, part_class
from ..parts.spec import ModelSpec, TensorSpec


def expected_tensors(spec: ModelSpec) -> list[TensorSpec]:
    """Every tensor the model reads, in checkpoint order (src/model_config.cpp:78-97)."""
    specs = part_class("embedding", spec.embedding).tensor_specs(spec.embedding, "")
    for layer in spec.layers:
        specs += part_class("block", layer.block).tensor_specs(layer.block, layer.prefix)
    specs += part_class("norm", spec.final_norm).tensor_specs(spec.final_norm, spec.final_norm["name"])
    specs += part_class("head", spec.head).tensor_specs(spec.head, "")
    return specs


def cache_needs(spec: ModelSpec) -> dict[int, CacheNeed]:
    """What each cache stream of the order list needs (decided by the run that writes it)."""
    needs: dict[int, CacheNeed] = {}
    for entry in spec.order:
        if entry.writes_cache:
            block = spec.layers[entry.layer].block
            needs[entry.cache] = part_class("block", block).cache_need(block)
    return needs


class DecoderModel:
    """Runs the tokens of one step through the parts.  It owns weights, not caches."""

    def __init__(self, spec: ModelSpec, weights, runtime: Runtime):
        spec.validate()
        self.spec = spec
        self.runtime = runtime
        self.embedding = build_part("embedding", spec.embedding, "", weights, runtime)
        self.blocks = [build_part("block", layer.block, layer.prefix, weights, runtime) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, spec.final_norm["name"], weights, runtime)
        self.head = build_part("head", spec.head, "", weights, runtime)
        self.cache_needs = cache_needs(spec)

    def forward(self, ctx, caches: dict[int, LayerCache]):
        """Logits (32-bit, [len(want_rows), vocab]) of the rows ``ctx.want_rows``."""
        hidden = self.forward_hidden(ctx, caches)
        return self.logits(hidden, ctx.want_rows)

    def forward_hidden(self, ctx, caches: dict[int, LayerCache]):
        residual = self.embedding.forward(ctx.token_ids)
        delta = None
        for entry in self.spec.order:
            cache = caches[entry.cache]
            if cache.writes != entry.writes_cache:
                cache = LayerCache(cache.need, entry.writes_cache, cache.pages, cache.block_table, cache.page_size, cache.state)
            residual, delta = self.blocks[entry.layer].forward(residual, delta, ctx, cache)
        if delta is not None:
            from .. import ops

            ops.add_(residual, delta)
        return residual

    def logits(self, residual, want_rows):
        if want_rows is None or want_rows.shape[0] == 0:
            return None
        from .. import ops

        if self.final_norm.supports_lazy and want_rows.shape[0] <= ops.fused_rows_limit(self.runtime.dtype, residual.device):
            return self.head.forward(self.final_norm.forward(residual, None, rows=want_rows, lazy=True))
        return self.head.forward(self.final_norm.forward(residual, None, rows=want_rows))
