"""Choosing the next token of every request that reached its last known token."""
from __future__ import annotations

import torch

from .. import ops


class Sampler:
    """Greedy, temperature and top-p selection on the device (app/server.cpp:237-277).

    Draw number ``k`` of a request uses the uniform number ``ops.uniform_from(seed, k)``,
    so what a request generates does not depend on the batch it ran in, nor on whether
    it was preempted and recomputed.
    """

    def __init__(self, device: torch.device):
        self.device = device

    def select(self, logits: torch.Tensor, params: list, draw_indices: list[int]) -> list[int]:
        """One token per row of ``logits`` (32-bit, [rows, vocab]); ``params[i]`` has temperature, top_p, seed."""
        rows = logits.shape[0]
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        if all(not p.temperature > 0.0 for p in params):
            ops.argmax(logits, out)
        else:
            host = torch.tensor([[p.temperature, p.top_p] for p in params], dtype=torch.float32)
            seeds = torch.tensor([[p.seed, k] for p, k in zip(params, draw_indices)], dtype=torch.int64)
            host, seeds = host.to(logits.device), seeds.to(logits.device)
            ops.sample(logits, host[:, 0].contiguous(), host[:, 1].contiguous(), seeds[:, 0].contiguous(), seeds[:, 1].contiguous(), out)
        tokens = out.cpu().tolist()                 # the host waits for the step here,
        ops.check_device_errors(logits.device)      # so this is where a fault a kernel recorded on the device surfaces
        return tokens
