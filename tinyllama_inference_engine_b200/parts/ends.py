"""The two ends of a model: token embedding and output head."""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, register_part
from .spec import PartSpec, TensorSpec


class TokenEmbedding(Part):
    """hidden = table[token], a row copy without scaling (src/model.cpp:94-97).

    params: ``vocab_size``, ``hidden_size``, ``name``.  The row is widened into the
    32-bit residual stream by a gather kernel (the reference copies one row per token
    with a device memcpy, src/cuda/model.cu:572-576).
    """

    capturable = True
    category = "embedding"

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(f"{spec['name']}.weight", (spec["vocab_size"], spec["hidden_size"]))]

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.table = weights.get(f"{spec['name']}.weight", runtime.dtype).contiguous()
        self.hidden = int(spec["hidden_size"])

    def forward(self, token_ids):
        residual = self.runtime.workspace.get("residual", token_ids.shape[0], self.hidden, torch.float32)
        ops.embedding(self.table, token_ids, residual)
        return residual


class LinearHead(Part):
    """logits = W . normed, 32-bit out, for the wanted rows only (src/model.cpp:217-225).

    params: ``vocab_size``, ``hidden_size``, ``name``, ``tied_to`` (name of the
    embedding table, or None).  With ``tied_to`` the head's own tensor is optional:
    a checkpoint that stores it anyway is read as it is, one that does not makes the
    head alias the embedding table.  The reference refuses tied checkpoints
    (src/model_config.cpp:72).
    """

    capturable = True
    category = "head"

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(f"{spec['name']}.weight", (spec["vocab_size"], spec["hidden_size"]), optional=bool(spec.get("tied_to")))]

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        own = f"{spec['name']}.weight"
        source = own if not spec.get("tied_to") or weights.has(own) else f"{spec['tied_to']}.weight"
        self.weight = weights.get(source, runtime.dtype).contiguous()
        self.vocab = int(spec["vocab_size"])

    def forward(self, normed_rows):
        """``normed_rows`` is the normalised hidden state of the wanted rows, or an ops.LazyNorm of it."""
        rows = normed_rows.shape[0]
        logits = torch.empty((rows, self.vocab), dtype=torch.float32, device=self.weight.device)
        if isinstance(normed_rows, ops.LazyNorm):
            ops.norm_linear(normed_rows, self.weight, logits)
        else:
            ops.linear(normed_rows, self.weight, logits)
        return logits


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "linear_head", LinearHead)
