"""The gated feed-forward."""
from __future__ import annotations

import torch

from .. import ops
from ..errors import ConfigError
from .base import FeedForward, register_part
from .spec import PartSpec, TensorSpec


class GatedMLP(FeedForward):
    """down( act(gate(x)) * up(x) ) with act = SiLU (src/model.cpp:187-203, src/operators.cpp:148-164).

    params: ``hidden_size``, ``intermediate_size``, ``activation`` ("silu").
    tensors: ``<prefix>.{gate,up}_proj.weight [inter, hidden]``,
    ``<prefix>.down_proj.weight [hidden, inter]``.  gate and up are stacked at load
    time into one ``[2 * inter, hidden]`` product; the activation and the product with
    ``up`` are computed in 32-bit.
    """

    capturable = True
    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, inter = spec["hidden_size"], spec["intermediate_size"]
        return [
            TensorSpec(f"{prefix}.gate_proj.weight", (inter, hidden)),
            TensorSpec(f"{prefix}.up_proj.weight", (inter, hidden)),
            TensorSpec(f"{prefix}.down_proj.weight", (hidden, inter)),
        ]

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        if spec.get("activation", "silu") != "silu":
            raise ConfigError(f"gated_mlp has no activation {spec.get('activation')!r}")
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        dtype = runtime.dtype
        self.w_gate_up = torch.cat([weights.get(f"{prefix}.gate_proj.weight", dtype), weights.get(f"{prefix}.up_proj.weight", dtype)], dim=0).contiguous()
        self.w_down = weights.get(f"{prefix}.down_proj.weight", dtype).contiguous()

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_down)

    def forward(self, x, ctx, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        act = ws.get("activated", tokens, self.inter, dtype)
        if tokens <= ops.fused_rows_limit(dtype, act.device):
            # few rows: the gate is applied in the first product's epilogue, the residual add in the second's
            if isinstance(x, ops.LazyNorm):
                ops.norm_linear(x, self.w_gate_up, act, gated=True)
            else:
                ops.linear_gated(x, self.w_gate_up, act)
        elif dtype == torch.bfloat16:
            ops.linear_gated(x.tensor() if isinstance(x, ops.LazyNorm) else x, self.w_gate_up, act)   # picks the fused kernel for its size
        else:
            if isinstance(x, ops.LazyNorm):
                x = x.tensor()
            gate_up = ws.get("gate_up", tokens, 2 * self.inter, dtype)
            ops.linear(x, self.w_gate_up, gate_up)
            ops.silu_mul(gate_up, act)
        if accumulate_into is not None:
            ops.linear_accumulate(act, self.w_down, accumulate_into, prepare)
            return None
        out = ws.get("ff_out", tokens, self.hidden, dtype)
        ops.linear(act, self.w_down, out)
        return out


register_part("feed_forward", "gated_mlp", GatedMLP)
