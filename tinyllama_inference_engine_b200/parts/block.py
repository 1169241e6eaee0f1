"""How the parts of one layer are arranged."""
from __future__ import annotations

from .base import Block, CacheNeed, LayerCache, build_part, norm_then_part, part_class, register_part
from .spec import PartSpec, TensorSpec


class PreNormResidualBlock(Block):
    """x -> x + mixer(norm(x)) -> x + feed_forward(norm(x))  (src/model.cpp:112-207).

    params: ``mixer``, ``feed_forward``, ``mixer_norm``, ``feed_forward_norm``
    (PartSpecs) and the tensor-name suffix of each (``*_name``).
    The hidden state travels as (32-bit residual, output not yet added): each norm
    adds the pending output into the residual before normalising, which is the
    reference's separate add kernel (src/cuda/kernels.cu:208-215) fused into its
    norm (:67-84).
    """

    _SLOTS = (("mixer_norm", "norm"), ("mixer", "mixer"), ("feed_forward_norm", "norm"), ("feed_forward", "feed_forward"))

    capturable = True

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        specs: list[TensorSpec] = []
        for slot, category in cls._SLOTS:
            child = spec[slot]
            specs += part_class(category, child).tensor_specs(child, f"{prefix}.{spec[slot + '_name']}")
        return specs

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        return part_class("mixer", spec["mixer"]).cache_need(spec["mixer"])

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        for slot, category in self._SLOTS:
            setattr(self, slot, build_part(category, spec[slot], f"{prefix}.{spec[slot + '_name']}", weights, runtime))

    accepts_next_norm = True

    @property
    def first_norm(self):
        return self.mixer_norm

    def forward(self, residual, pending, ctx, cache: LayerCache, next_norm=None):
        from .. import ops

        fused = residual.shape[0] <= ops.fused_rows_limit(self.runtime.dtype, residual.device)
        pending = norm_then_part(self.mixer_norm, self.mixer, residual, pending, fused, self.feed_forward_norm, ctx, cache)
        pending = norm_then_part(self.feed_forward_norm, self.feed_forward, residual, pending, fused, next_norm, ctx)
        return residual, pending


register_part("block", "pre_norm_residual", PreNormResidualBlock)
