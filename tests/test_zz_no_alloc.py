"""The decode-attention entry point for callers that cannot allocate device memory.

Some users of these kernels may not call cudaMalloc at all: they run inside a host application that gave them a
fixed memory budget, or inside a loop where an allocation could stall the device, or next to a framework whose
allocator is not theirs to use.  They pass inputs and outputs they already own; the split-KV scratch (partial
results and arrival counters) they cannot provide, so ``tlie_decode_attention_static`` keeps it in an array built
into the library.  This test calls that function through its exported C symbol, twice in a row on the same
inputs, and checks each result against the ordinary entry point (which takes its scratch from the caller) and
against the plain attention of tests/plain_ops.py; the device's free memory is read before and after the two
calls, so an allocation inside them would show.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import numpy as np
import pytest
import torch

import plain_ops

pytestmark = pytest.mark.gpu


def _case(seed: int, requests: int, q_heads: int, kv_heads: int, head_dim: int, page_size: int, lengths):
    rng = np.random.default_rng(seed)
    torch.manual_seed(seed)
    pages_per = [-(-n // page_size) for n in lengths]
    num_pages = sum(pages_per) + 2
    order = rng.permutation(num_pages)
    table = -np.ones((requests, max(pages_per) + 1), dtype=np.int32)
    at = 0
    for i, n in enumerate(pages_per):
        table[i, :n] = order[at : at + n]
        at += n
    pages = (torch.randn(num_pages, 2, kv_heads, page_size, head_dim) * 0.5).bfloat16().cuda()
    qkv = (torch.randn(requests, (q_heads + 2 * kv_heads) * head_dim) * 0.5).bfloat16().cuda()
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32).cuda()
    return qkv, pages, positions, torch.from_numpy(table).cuda()


@pytest.mark.parametrize("splits", [1, 6])
def test_static_scratch_entry_point_matches_the_ordinary_one(splits):
    from tinyllama_inference_engine_b200.ops import fast

    requests, q_heads, kv_heads, head_dim, page_size = 5, 32, 4, 64, 64
    lib = fast.decode_attention_library(head_dim)
    qkv, pages, positions, table = _case(31, requests, q_heads, kv_heads, head_dim, page_size, [1, 64, 333, 1500, 129])
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)

    def arguments(out, scratch=None):
        head = [c_void_p(qkv.data_ptr()), c_int(qkv.shape[1]), c_void_p(pages.data_ptr()), c_void_p(positions.data_ptr()),
                c_void_p(table.data_ptr()), c_int(table.shape[1]), c_void_p(out.data_ptr())]
        if scratch is not None:
            head.append(c_void_p(scratch.data_ptr()))
        return head + [c_int(requests), c_int(q_heads), c_int(kv_heads), c_int(page_size), c_int(0), c_float(head_dim ** -0.5),
                       c_int(splits), c_int(0), c_void_p(0), c_int(0), stream]

    floats = lib.tlie_decode_attention_scratch_floats(c_int(requests), c_int(q_heads), c_int(splits))
    scratch = torch.zeros(floats, dtype=torch.float32, device="cuda")
    want = torch.empty(requests, q_heads * head_dim, dtype=torch.bfloat16, device="cuda")
    assert lib.tlie_decode_attention(*arguments(want, scratch)) == 0
    torch.cuda.synchronize()
    assert bool(torch.isfinite(want.float()).all())
    plain = torch.empty(requests, q_heads * head_dim)
    plain_ops.paged_attention(qkv.cpu(), pages.cpu(), positions.cpu(), torch.arange(requests, dtype=torch.int32), table.cpu(), plain,
                              q_heads, kv_heads, head_dim, page_size)
    assert float((want.float().cpu() - plain).abs().max()) <= 1.6e-2
    outputs = [torch.full_like(want, float("nan")) for _ in range(2)]   # made before free memory is read
    lib.tlie_decode_attention_static(*arguments(outputs[0]))            # set-up call: the array's address is looked up once per device
    torch.cuda.synchronize()
    outputs[0].fill_(float("nan"))
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for call, got in enumerate(outputs):   # the second call finds the array as the first one left it
        assert lib.tlie_decode_attention_static(*arguments(got)) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "device memory was allocated or freed inside the calls"
    for call, got in enumerate(outputs):
        assert float((got.float() - want.float()).abs().max()) <= 1.6e-2, f"call {call}"
        assert float((got.float().cpu() - plain).abs().max()) <= 1.6e-2, f"call {call} against the plain attention"


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from tinyllama_inference_engine_b200.ops import fast

    lib = fast.decode_attention_library(64)
    requests, q_heads, kv_heads = 64, 32, 4
    qkv, pages, positions, table = _case(32, requests, q_heads, kv_heads, 64, 64, [70] * requests)
    out = torch.zeros(requests, q_heads * 64, dtype=torch.bfloat16, device="cuda")
    status = lib.tlie_decode_attention_static(
        c_void_p(qkv.data_ptr()), c_int(qkv.shape[1]), c_void_p(pages.data_ptr()), c_void_p(positions.data_ptr()), c_void_p(table.data_ptr()),
        c_int(table.shape[1]), c_void_p(out.data_ptr()), c_int(requests), c_int(q_heads), c_int(kv_heads), c_int(64), c_int(0), c_float(0.125),
        c_int(8), c_int(0), c_void_p(0), c_int(0), c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert status == 1  # cudaErrorInvalidValue: 64 * 32 * 8 triples are more than the built-in array holds
    assert float(out.float().abs().max()) == 0.0  # nothing was launched
    # head counts no launch can have are refused before anything (the clearing of the counters included) is enqueued
    for q, kv in ((32, 0), (32, 5), (0, 4), (34, 2)):
        status = lib.tlie_decode_attention_static(
            c_void_p(qkv.data_ptr()), c_int(qkv.shape[1]), c_void_p(pages.data_ptr()), c_void_p(positions.data_ptr()), c_void_p(table.data_ptr()),
            c_int(table.shape[1]), c_void_p(out.data_ptr()), c_int(2), c_int(q), c_int(kv), c_int(64), c_int(0), c_float(0.125),
            c_int(1), c_int(0), c_void_p(0), c_int(0), c_void_p(torch.cuda.current_stream().cuda_stream))
        assert status == 1, (q, kv)
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0
