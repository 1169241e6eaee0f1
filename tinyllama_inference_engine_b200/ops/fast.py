"""The bfloat16 serving kernels: tensor-core matrix products and attention.

Kept apart from the core set because they are specialised (by head size, by shape)
and compiled only for what a model needs.
"""
from __future__ import annotations

import torch

from ..errors import KernelError

library_gemm_calls = 0  # vendor-library matrix products issued (not this engine's kernels)


def build_all() -> list:
    return []


def linear_bf16(x, weight, out) -> None:
    global library_gemm_calls
    if weight.dtype != torch.bfloat16 or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("linear: the bfloat16 path takes bfloat16 weights", code="invalid_dtype")
    library_gemm_calls += 1
    if out.dtype == torch.float32:
        torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
    else:
        torch.mm(x, weight.t(), out=out)


def paged_attention_bf16(qkv, pages, positions, token_seq, block_table, out, q_heads, kv_heads, head_dim, page_size, window, scale, batch) -> bool:
    """Run a specialised kernel if one covers this shape; False sends the caller to the general one."""
    return False
