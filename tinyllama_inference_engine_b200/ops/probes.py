"""Measurements behind the kernels' designs, for ``kernel-bench --probes`` and ``kernel-bench --attention-phases``.

``hardware_probes`` runs the loops of ``csrc/probes.cu``: what a ``tcgen05.mma`` of a given shape costs the tensor core, what
the hand-off primitives cost a lone thread, how fast a warp gets through the arithmetic of a softmax tile.
``attention_phase_cycles`` builds the tensor-memory prompt attention with its cycle counters compiled in (one build per
phase: ``-DTLIE_ATTN_TIMELINE -DTLIE_ATTN_TIMELINE_SLOT=k``) and reports where a key tile's cycles go in each role of one CTA.
Nothing of the engine's product path calls either.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import torch

from .build import load_library

SOFTMAX_PHASES = ["loop and what follows the arrival", "wait for the scores", "load them from tensor memory", "mask, maximum, reference",
                  "64 x (multiply-add, exp2, add), 32 packs", "P into tensor memory, its wait, arrival"]
SCORE_ISSUER_PHASES = ["loop", "wait for Q and K", "wait for the S buffer (the product that read its P)", "issue the score MMAs, commit"]
PRODUCER_PHASES = ["page lookup, issue of the copies", "wait for a free buffer"]


def hardware_probes(device: torch.device | str = "cuda:0") -> dict:
    from .. import ops

    device = torch.device(device)
    lib = load_library("tlie_probes", ["probes.cu"])
    flag = ops.error_flag(device)
    stream = ops._stream()
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    out = torch.zeros(4 * sms, dtype=torch.int64, device=device)
    report: dict = {"sms": sms, "mma_cycles": {}, "handoff_cycles": {}, "arithmetic_cycles_per_64_values": {}}

    def mma(blocks: int, n: int, chain: int, straight: int) -> float:
        ops._check(lib.tlie_probe_mma(c_int(blocks), c_int(n), c_int(chain), c_int(straight), c_void_p(out.data_ptr()), ops._ptr(flag), stream), "probe_mma")
        torch.cuda.synchronize(device)
        ops.check_device_errors(device)
        return float(out[0 : 2 * blocks : 2].double().mean())

    for blocks, per_sm in ((sms, "one CTA per SM"), (2 * sms, "two CTAs per SM")):
        for straight, how in ((1, "straight-line issue"), (0, "one MMA per loop turn")):
            for n in (32, 64, 128, 256):
                mma(blocks, n, 64, straight)
                short, long = mma(blocks, n, 256, straight), mma(blocks, n, 1280, straight)
                report["mma_cycles"][f"128 x {n} x 16, {how}, {per_sm}"] = round((long - short) / 1024, 1)
    five = torch.zeros(5, dtype=torch.int64, device=device)
    ops._check(lib.tlie_probe_handoff(c_void_p(five.data_ptr()), ops._ptr(flag), stream), "probe_handoff")
    torch.cuda.synchronize(device)
    ops.check_device_errors(device)
    names = ["arrive + wait on the barrier just completed", "wait on a completed barrier", "tcgen05.commit, nothing outstanding",
             "tcgen05.commit + wait for its arrival", "fence.proxy.async"]
    report["handoff_cycles"] = dict(zip(names, five.tolist()))
    values = (torch.rand(4096, device=device) * 4 - 6).contiguous()
    sink = torch.zeros(sms * 256, device=device)
    cycles = torch.zeros(1, dtype=torch.int64, device=device)
    for threads, where in ((128, "one warp per scheduler"), (256, "two warps per scheduler")):
        for mode, what in ((0, "64 exp2"), (1, "64 multiply-adds and 64 adds")):
            for _ in range(2):
                ops._check(lib.tlie_probe_arithmetic(c_int(mode), c_int(sms), c_int(threads), ops._ptr(values), ops._ptr(sink), c_void_p(cycles.data_ptr()), c_int(50), stream),
                           "probe_arithmetic")
                torch.cuda.synchronize(device)
            report["arithmetic_cycles_per_64_values"][f"{what}, {where}"] = int(cycles)
    return report


def attention_phase_cycles(tokens: int, q_heads: int, kv_heads: int, head_dim: int, device: torch.device | str = "cuda:0") -> dict:
    """Cycles per key tile of one thread of each role of CTA (0, 0), for one request of ``tokens`` tokens (a multiple of 128) attending to itself."""
    from .. import ops
    from . import fast

    device = torch.device(device)
    page = 64
    pages = -(-tokens // page)
    qkv = torch.randn(tokens, (q_heads + 2 * kv_heads) * head_dim, device=device).bfloat16()
    pool = torch.randn(pages, 2, kv_heads, page, head_dim, device=device).bfloat16()
    table = torch.arange(pages, dtype=torch.int32, device=device).view(1, pages).contiguous()
    tiles = torch.tensor(fast.paired_attention_tiles([tokens], [0], [0]), dtype=torch.int32, device=device).view(-1, 4)
    starts = torch.tensor([0, tokens], dtype=torch.int32, device=device)
    first = torch.zeros(1, dtype=torch.int32, device=device)
    out = torch.empty(tokens, q_heads * head_dim, device=device, dtype=torch.bfloat16)
    roles = ((0, "softmax thread", SOFTMAX_PHASES), (8, "score issuer", SCORE_ISSUER_PHASES), (16, "producer", PRODUCER_PHASES))
    report = {role: {"phases": {}} for _, role, _ in roles}
    for slot in range(-1, 6):
        defines = {"TLIE_ATTN_TIMELINE": 1} if slot < 0 else {"TLIE_ATTN_TIMELINE": 1, "TLIE_ATTN_TIMELINE_SLOT": slot}
        lib = load_library("tlie_attn_prefill_tc_phase%s" % ("_all" if slot < 0 else slot), ["attention_prefill_tc.cu"], defines)
        for _ in range(5):
            ops._check(lib.tlie_prefill_attention_tc(ops._ptr(qkv), c_int(qkv.shape[1]), c_int(tokens), ops._ptr(pool), c_int(pages), ops._i32(tiles, "tiles"), c_int(tiles.shape[0]),
                                                     ops._i32(starts, "seq_starts"), ops._i32(first, "first_positions"), ops._i32(table, "block_table"), c_int(pages), ops._ptr(out),
                                                     c_int(q_heads), c_int(kv_heads), c_int(head_dim), c_int(page), c_int(0), c_float(head_dim ** -0.5),
                                                     ops._ptr(ops.error_flag(device)), ops._stream()), "prefill_attention_tc")
        torch.cuda.synchronize(device)
        ops.check_device_errors(device)
        stamps = (ctypes.c_longlong * 24)()
        ops._check(lib.tlie_prefill_attention_tc_timeline(stamps), "prefill_attention_tc_timeline")
        for base, role, phases in roles:
            tiles_run = max(1, stamps[base + 7])
            if slot < 0:
                report[role]["tiles"] = int(stamps[base + 7])
                report[role]["cycles_per_tile"] = round(stamps[base + 6] / tiles_run)
            elif slot < len(phases):
                report[role]["phases"][phases[slot]] = round(stamps[base + slot] / tiles_run)
    return report


def product_comparison(rows: int, hidden: int, intermediate: int, qkv_width: int, device: torch.device | str = "cuda:0", launches: int = 12) -> dict:
    """The four products of a layer for a step of ``rows`` rows (128 or more), bfloat16: the engine's own tcgen05 kernels (tiles on one
    SM, tiles on pairs of SMs; plain, adding into the 32-bit residual, gated) against the library's product plus the small kernel
    the fused form saves.  Microseconds per launch inside a replayed CUDA graph, every launch with another copy of the weights so
    that they come from HBM.  Each form runs with the tile width the engine would pick for it; ``own_runs`` says which form a step of
    this size gets (ops.fast.tcgen05_takes, pair_tiles_pay)."""
    from .. import ops
    from . import fast

    device = torch.device(device)

    def timed(call) -> float:
        for index in range(3):
            call(index)
        torch.cuda.synchronize(device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for index in range(launches):
                call(index)
        graph.replay()
        torch.cuda.synchronize(device)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize(device)
        return round(start.elapsed_time(end) / launches * 1e3, 1)

    report = {}
    for name, N, K, kind in (("qkv", qkv_width, hidden, "plain"), ("o", hidden, hidden, "add"), ("gate_up", 2 * intermediate, hidden, "gated"),
                             ("down", hidden, intermediate, "add")):
        copies = max(2, int(300e6 / (N * K * 2)))
        x = torch.randn(rows, K, device=device).bfloat16()
        weights = [(torch.randn(N, K, device=device) * 0.05).bfloat16() for _ in range(copies)]
        out = torch.empty(rows, N, device=device, dtype=torch.bfloat16)
        line = {"N": N, "K": K}
        if kind == "plain":
            line["library"] = timed(lambda i: torch.mm(x, weights[i % copies].t(), out=out))
            line["own, one SM"] = timed(lambda i: fast.gemm_tcgen05(x, weights[i % copies], out, pair=False))
            line["own, SM pairs"] = timed(lambda i: fast.gemm_tcgen05(x, weights[i % copies], out, pair=True))
            line["own_runs"] = fast.tcgen05_takes(rows, N, K) and ("SM pairs" if fast.pair_tiles_pay(rows, N) else "one SM")
        elif kind == "add":
            residual = torch.zeros(rows, N, device=device)
            line["library + add kernel"] = timed(lambda i: (torch.mm(x, weights[i % copies].t(), out=out), ops.add_(residual, out)))
            line["own, one SM"] = timed(lambda i: fast.gemm_tcgen05_accumulate(x, weights[i % copies], residual, pair=False))
            line["own, SM pairs"] = timed(lambda i: fast.gemm_tcgen05_accumulate(x, weights[i % copies], residual, pair=True))
            line["own_runs"] = fast.can_accumulate(rows, weights[0]) and ("SM pairs" if fast.use_sm_pairs and rows >= fast.PAIR_MIN_ROWS else "one SM")
        else:
            half = torch.empty(rows, N // 2, device=device, dtype=torch.bfloat16)
            line["library + activation kernel"] = timed(lambda i: (torch.mm(x, weights[i % copies].t(), out=out), ops.silu_mul(out, half)))
            line["own, one SM"] = timed(lambda i: fast.gemm_tcgen05_gated(x, weights[i % copies], half, pair=False))
            line["own, SM pairs"] = timed(lambda i: fast.gemm_tcgen05_gated(x, weights[i % copies], half, pair=True))
            line["own_runs"] = fast.gated_takes(rows, N, K) and ("SM pairs" if fast.use_sm_pairs and (rows >= fast.PAIR_MIN_ROWS or (rows >= 512 and rows % 256 == 0)) else "one SM")
        report[name] = line
        del weights
    ops.check_device_errors(device)
    return report
