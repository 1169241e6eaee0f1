"""Rotary position encoding as a part."""
from __future__ import annotations

import numpy as np
import torch

from .base import PositionEncoding, register_part


class RotaryEmbedding(PositionEncoding):
    """Half-split rotation of q and k (src/operators.cpp:47-78).

    params: ``rotary_dim`` (how many leading elements of a head rotate; the reference
    rotates the whole head), ``theta``.  The frequency of pair d is
    ``theta ** (-2 d / rotary_dim)`` evaluated in 32-bit, as the reference's ``std::pow``
    on floats does; the angle ``float(position) * frequency`` and its sine and cosine
    are 32-bit inside the kernel.  Keys are cached after rotation, so the cache never
    depends on this part.
    """

    capturable = True

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.rotary_dim = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        half = self.rotary_dim // 2
        exponent = (np.float32(-2.0) * np.arange(half, dtype=np.float32)) / np.float32(self.rotary_dim)
        inv_freq = np.power(np.float32(self.theta), exponent, dtype=np.float32)
        self.inv_freq = torch.from_numpy(inv_freq).to(runtime.device)

    def rotary_table(self):
        return self.inv_freq, self.rotary_dim


class NoPositionEncoding(PositionEncoding):
    """Leaves q and k as they are (a mixer that needs no positions)."""

    capturable = True

    def rotary_table(self):
        return None

    def apply(self, qkv, ctx, q_heads, kv_heads, head_dim) -> None:
        return None


register_part("position", "rotary", RotaryEmbedding)
register_part("position", "none", NoPositionEncoding)
