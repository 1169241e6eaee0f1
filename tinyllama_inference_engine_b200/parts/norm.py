"""RMSNorm, with the residual add fused in front of it."""
from __future__ import annotations

import torch

from .. import ops
from .base import Norm, register_part
from .spec import PartSpec, TensorSpec


class RMSNorm(Norm):
    """y = x / sqrt(mean(x^2) + eps) * weight, eps inside the root (src/operators.cpp:22-45).

    params: ``size``, ``eps``.  tensors: ``<prefix>.weight [size]``.
    The statistics, the scale and the residual sum are 32-bit in both precisions;
    the weight is held in 32-bit (exact for a bfloat16 checkpoint).
    """

    capturable = True
    supports_lazy = True

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(f"{prefix}.weight", (spec["size"],), init="norm", std=0.1)]

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight = weights.get(f"{prefix}.weight", torch.float32).contiguous()

    def forward(self, residual, delta=None, rows=None, lazy: bool = False):
        """``lazy`` (and nothing to add): hand the norm on to the product that consumes it (ops.LazyNorm)."""
        if lazy and delta is None:
            handle = ops.LazyNorm(residual, self.weight, self.eps, rows, lambda: self.forward(residual, None, rows))
            if rows is None and self.runtime.dtype == torch.bfloat16:
                # where a product that completes the residual may leave this norm's input (ops.linear_accumulate(..., prepare=handle))
                ws = self.runtime.workspace
                handle.buffers = (ws.get("prepared_norm", residual.shape[0], self.size, torch.bfloat16),
                                  ws.get("prepared_squares", residual.shape[0], -(-self.size // 16), torch.float32))
            return handle
        count = residual.shape[0] if rows is None else rows.shape[0]
        out = self.runtime.workspace.get("normed" if rows is None else "normed_rows", count, self.size, self.runtime.dtype)
        ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows)
        return out


register_part("norm", "rmsnorm", RMSNorm)
