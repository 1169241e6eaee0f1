"""A decoder assembled from a ModelSpec: embedding, the ordered runs of blocks, norm, head."""
from __future__ import annotations

from ..parts.base import CacheNeed, LayerCache, Runtime, build_part, capturable, part_class
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
        # whether a step through this model may be captured as a CUDA graph: every part has to vouch for itself
        self.capturable = all(capturable(part) for part in [self.embedding, *self.blocks, self.final_norm, self.head])

    def forward(self, ctx, caches: dict[int, LayerCache], trace: dict | None = None):
        """Logits (32-bit, [len(want_rows), vocab]) of the rows ``ctx.want_rows``.

        ``trace``: a dictionary that receives the hidden state of all rows after every run of a layer (32-bit copies)."""
        hidden, pending = self._run_blocks(ctx, caches, trace)
        return self.logits(hidden, ctx.want_rows, pending if ctx.wants_every_row_in_order else None)

    def forward_hidden(self, ctx, caches: dict[int, LayerCache]):
        return self._run_blocks(ctx, caches)[0]

    def _run_blocks(self, ctx, caches: dict[int, LayerCache], trace: dict | None = None):
        """The complete residual stream of the step's rows, and a lazy final norm of it if the last block left one prepared."""
        from .. import ops

        residual = self.embedding.forward(ctx.token_ids)
        pending = None
        order = self.spec.order
        for index, entry in enumerate(order):
            cache = caches[entry.cache]
            if cache.writes != entry.writes_cache:
                cache = LayerCache(cache.need, entry.writes_cache, cache.pages, cache.block_table, cache.page_size, cache.state, cache.plane_pages)
            block = self.blocks[entry.layer]
            if block.accepts_next_norm:
                # the norm that reads this block's result: the next block's first one (if it names one), or the final norm
                following = self.blocks[order[index + 1].layer].first_norm if index + 1 < len(order) else self.final_norm
                residual, pending = block.forward(residual, pending, ctx, cache, next_norm=following)
            else:
                if isinstance(pending, ops.LazyNorm):
                    pending = None   # the residual is complete; this block does not know prepared norms
                residual, pending = block.forward(residual, pending, ctx, cache)
            if trace is not None:
                # the layer's output is the residual with what is still pending on it (a prepared norm means nothing is)
                complete = residual if pending is None or isinstance(pending, ops.LazyNorm) else residual + pending.float()
                trace[f"layer{index}.output"] = complete.float().clone()
        if isinstance(pending, ops.LazyNorm):
            return residual, pending
        if pending is not None:
            ops.add_(residual, pending)
        return residual, None

    def logits(self, residual, want_rows, prepared=None):
        """``prepared``: a lazy final norm of all rows that the last block left ready, usable when every row is wanted in order."""
        if want_rows is None or want_rows.shape[0] == 0:
            return None
        from .. import ops

        if self.final_norm.supports_lazy and want_rows.shape[0] <= ops.fused_rows_limit(self.runtime.dtype, residual.device):
            if prepared is not None and prepared.weight is self.final_norm.weight and prepared.shape[0] == want_rows.shape[0]:
                return self.head.forward(prepared)
            return self.head.forward(self.final_norm.forward(residual, None, rows=want_rows, lazy=True))
        return self.head.forward(self.final_norm.forward(residual, None, rows=want_rows))
