"""The engine's host logic (cache manager, batch packing, step function, model assembly) on the CPU.

The kernel wrappers are replaced by the plain per-kernel functions of tests/plain_ops.py,
so these tests say nothing about the kernels; they show that pages, block tables,
positions and wanted rows are right under every way of cutting the work.
"""
from __future__ import annotations

import pytest
import torch

import plain_llama
import plain_ops
import trace_tools
from tinyllama_inference_engine_b200 import EngineConfig
from tinyllama_inference_engine_b200.engine.runner import ModelRunner
from tinyllama_inference_engine_b200.errors import BatchError, KernelError, OutOfPages


def _runner(folder, max_tokens=1024, page_size=16, dtype="float32", max_batch_tokens=2048):
    config = EngineConfig(dtype=dtype, page_size=page_size, max_cache_tokens=max_tokens, max_requests=8, max_batch_tokens=max_batch_tokens, device="cpu", poison_freed_pages=True)
    return ModelRunner(folder, config)


def _full_logits(folder, requests):
    config, weights = plain_llama.load_model(folder)
    return {rid: plain_llama.forward(config, weights, tokens) for rid, tokens in requests.items()}


def test_without_kernels_the_engine_refuses_cpu_tensors(model_folders):
    runner = _runner(model_folders["a"])
    from tinyllama_inference_engine_b200.engine.batch import StepEntry

    with pytest.raises(KernelError, match="no CPU path"):
        runner.step([StepEntry("x", [1, 2, 3], [2])])


@pytest.mark.parametrize("key", ["a", "b", "c"])
def test_every_cut_gives_the_plain_logits(model_folders, monkeypatch, key):
    plain_ops.install(monkeypatch)
    folder = model_folders[key]
    vocab = plain_llama.load_model(folder)[0]["vocab_size"]
    requests = trace_tools.make_requests(vocab, [1, 7, 33, 70, 50, 41], seed=1)
    full = _full_logits(folder, requests)
    for steps in (trace_tools.whole(requests), trace_tools.tail_decode(requests), trace_tools.portions(requests)):
        runner = _runner(folder)
        worst = trace_tools.run_and_compare(runner, steps, full, atol=2e-5)
        runner.cache.check()
        assert not runner.cache.records and worst < 2e-5
    steps, peak = trace_tools.mixed(requests, seed=3, page_size=16)
    runner = _runner(folder, max_tokens=peak)
    trace_tools.run_and_compare(runner, steps, full, atol=2e-5)
    runner.cache.check()
    stats = runner.cache.stats()["groups"][0]
    assert stats["reuses"] > 0 and stats["free"] == stats["pages"]


def test_step_refuses_bad_batches(model_folders, monkeypatch):
    plain_ops.install(monkeypatch)
    from tinyllama_inference_engine_b200.engine.batch import StepEntry

    runner = _runner(model_folders["a"], max_tokens=32)
    with pytest.raises(BatchError, match="outside the vocabulary"):
        runner.step([StepEntry("x", [1, 9999], [])])
    with pytest.raises(BatchError, match="twice"):
        runner.step([StepEntry("x", [1], []), StepEntry("x", [2], [])])
    with pytest.raises(BatchError, match="wants place"):
        runner.step([StepEntry("x", [1, 2], [2])])
    with pytest.raises(BatchError, match="context"):
        runner.step([StepEntry("x", [1] * 129, [])])
    with pytest.raises(OutOfPages):
        runner.step([StepEntry("x", [1] * 40, [])])
    assert not runner.cache.records  # a refused step leaves nothing behind
    runner.step([StepEntry("x", [1] * 30, [29])])
    with pytest.raises(OutOfPages):
        runner.step([StepEntry("y", [1] * 10, [])])
    assert list(runner.cache.records) == ["x"]
    runner.finish("x")
    runner.cache.check()
    # the workspace's buffers have fixed addresses (captured graphs point at them): a step beyond the token budget is refused
    small = _runner(model_folders["a"], max_batch_tokens=8)
    with pytest.raises(BatchError, match="max_batch_tokens"):
        small.step([StepEntry("x", [1] * 5, []), StepEntry("y", [1] * 4, [])])
    assert not small.cache.records
    small.step([StepEntry("x", [1] * 5, []), StepEntry("y", [1] * 3, [2])])
    with pytest.raises(BatchError, match="workspace"):
        small.runtime.workspace.get("anything", 9, 4, torch.float32)


def test_own_products_run_where_their_tiles_fill_the_waves():
    from tinyllama_inference_engine_b200.ops import fast

    # 1.1B widths: the step of 2,048 rows, not the smaller ones
    assert fast.tcgen05_takes(2048, 2560, 2048) and fast.tcgen05_takes(2048, 2048, 2048, adding=True) and fast.tcgen05_takes(2048, 2048, 5632, adding=True)
    assert not fast.tcgen05_takes(1536, 2560, 2048) and not fast.tcgen05_takes(1024, 2560, 2048)   # small products: the library's start and end are shorter
    assert not fast.tcgen05_takes(1536, 2048, 5632, adding=True)        # 48 tiles for 74 pairs
    assert fast.tcgen05_takes(1792, 2048, 5632, adding=True)            # 56 tiles
    assert fast.tcgen05_takes(8192, 2560, 2048)
    # 7B / 8B widths: from 1,024 rows on
    assert fast.tcgen05_takes(1024, 12288, 4096) and fast.tcgen05_takes(1024, 4096, 4096, adding=True) and fast.tcgen05_takes(1536, 4096, 11008, adding=True)
    assert fast.tcgen05_takes(1280, 4096, 11008, adding=True)           # 55 tiles of 384 columns for 74 pairs
    assert fast.tcgen05_takes(8192, 4096, 14336, adding=True) and fast.tcgen05_takes(8192, 6144, 4096)
    assert not fast.tcgen05_takes(512, 12288, 4096) and not fast.tcgen05_takes(64, 32000, 2048)   # below the smallest row count
    # the gated product: from 1,024 rows, and from 512 where it is a large one
    assert fast.gated_takes(1024, 11264, 2048) and not fast.gated_takes(896, 11264, 2048) and fast.gated_takes(512, 22016, 4096) and not fast.gated_takes(384, 28672, 4096)


def test_gemm_tile_width_prefers_full_waves():
    """Waves of 148 persistent CTAs x tile width: the product whose 256-wide tiles fill one wave and a sliver gets one wave of
    320-wide tiles, or narrower tiles where that is no single wave either."""
    from tinyllama_inference_engine_b200.ops import fast

    assert fast.gemm_tile_width(2048, 2560) == 288      # 160 tiles of 256 would be two waves; 144 tiles of 288 are one
    assert fast.gemm_tile_width(2048, 2816) == 320      # 160 tiles of 288 are two waves; 144 tiles of 320 are one
    assert fast.gemm_tile_width(4096, 2560) == 256      # 256 tiles of 320 are no single wave, so the wide tile is no candidate
    assert not fast.pair_tiles_pay(2048, 2560)          # one wave on single SMs: it stays there
    # pairs of SMs: where waves of tiles make L2 the limit, or where a wide tile of theirs makes one wave of two
    assert fast.pair_tiles_pay(2048, 12288) and fast.gemm_tile_width(2048, 12288, pair=True) == 256
    assert fast.pair_tiles_pay(2048, 4096) and fast.gemm_tile_width(2048, 4096, pair=True) == 480       # 72 tiles for 74 pairs
    assert fast.gemm_tile_width(2048, 4096, pair=True, adding=True) == 480 and fast.gemm_tile_width(2048, 2048, pair=True, adding=True) == 256
    assert fast.gemm_tile_width(4096, 4096, pair=True, adding=True) == 256                             # no single wave: two accumulators
    assert not fast.pair_tiles_pay(512, 12288)          # below the pairs' row count
    assert fast.gemm_tile_width(2048, 2048) == 256      # 128 tiles: one wave
    assert fast.gemm_tile_width(256, 2048) == 128       # few row blocks: narrow tiles keep more CTAs busy
    for rows in (128, 300, 5000):
        for cols in (64, 1000, 32000):
            assert fast.gemm_tile_width(rows, cols) in fast.GEMM_TILE_WIDTHS + fast.GEMM_WIDE_TILES


def test_decode_attention_parts_fit_one_wave():
    """requests x kv heads x parts never exceeds the SMs while a (request, kv head) has a CTA to itself: no second wave."""
    from tinyllama_inference_engine_b200.ops import fast

    for requests in (1, 2, 3, 7, 8, 9, 16, 33, 37, 64):
        for kv_heads in (1, 2, 4, 8):
            parts = fast.decode_splits(requests, kv_heads, 4096)
            assert 1 <= parts <= 32
            if requests * kv_heads <= fast.sm_count():
                assert requests * kv_heads * parts <= fast.sm_count()
    assert fast.decode_splits(8, 4, 2048) == 4 and fast.decode_splits(1, 4, 2048) == 8 and fast.decode_splits(1, 4, 100) == 1


def test_block_lets_a_part_add_to_the_residual_in_steps_of_many_rows(monkeypatch):
    """The block's choice, with stand-in parts: few rows -> norm and add go into the part's kernels (lazy norm, accumulate_into);
    many rows -> a materialised norm, and accumulate_into only if the part says it can add for that many rows."""
    from tinyllama_inference_engine_b200 import ops
    from tinyllama_inference_engine_b200.parts import norm_then_part

    monkeypatch.setattr(ops, "fused_rows_limit", lambda dtype, device: 16)
    calls = []

    class Norm:
        supports_lazy = True
        weight, eps = object(), 1e-5

        def forward(self, residual, delta, lazy=False):
            calls.append(("norm", delta is not None, lazy))
            return "lazy" if lazy else "normed"

    class Part:
        accepts_lazy_norm = fuses_residual_add = True
        prepares_next_norm = False

        def __init__(self, adds):
            self.adds = adds

        def adds_to_residual(self, rows):
            return self.adds

        def forward(self, x, accumulate_into=None):
            calls.append(("part", x, accumulate_into is not None))
            return None if accumulate_into is not None else "out"

    few, many = torch.zeros(8, 4), torch.zeros(200, 4)
    assert norm_then_part(Norm(), Part(False), few, None, True, None) is None
    assert calls == [("norm", False, True), ("part", "lazy", True)]
    calls.clear()
    assert norm_then_part(Norm(), Part(False), many, "pending", False, None) == "out"
    assert calls == [("norm", True, False), ("part", "normed", False)]
    calls.clear()
    assert norm_then_part(Norm(), Part(True), many, "pending", False, None) is None
    assert calls == [("norm", True, False), ("part", "normed", True)]


def test_the_engine_refuses_weights_with_another_digest(model_folders):
    """EngineConfig.weights_sha256 pins the model folder's weights (the reference: src/weight_store.cpp:150-190)."""
    from tinyllama_inference_engine_b200.errors import EngineError
    from tinyllama_inference_engine_b200.weights import weights_sha256

    folder = model_folders["a"]
    good = weights_sha256(folder)
    ModelRunner(folder, EngineConfig(dtype="float32", page_size=16, max_cache_tokens=64, device="cpu", weights_sha256=good))
    with pytest.raises(EngineError) as caught:
        ModelRunner(folder, EngineConfig(dtype="float32", page_size=16, max_cache_tokens=64, device="cpu", weights_sha256="f" * 64))
    assert caught.value.code == "checksum_mismatch"


def test_a_packed_step_holds_what_its_entries_say():
    """The packer's flat buffer, section by section, against plain loops: decoding requests beside prompt portions, wanted places,
    block tables of two page groups, a registered work list; written fresh and into a buffer of fixed address."""
    from tinyllama_inference_engine_b200.engine.batch import StepEntry, StepPlan, pack_step, register_step_plan, unregister_step_plan

    entries = [StepEntry("d0", [7], [0]), StepEntry("d1", [9], []), StepEntry("p0", [3, 1, 4, 1, 5], [4, 0]), StepEntry("p1", [2, 6], [1])]
    firsts, slots = [40, 3, 0, 17], [5, 0, 2, 9]
    tables = [[[1, 2, -1], [3, -1, -1], [4, 5, 6], [7, -1, -1]], [[8, -1, -1], [9, -1, -1], [10, 11, -1], [12, 13, -1]]]
    register_step_plan(StepPlan("test_lengths_twice", 2, lambda q, f, s: [n for n in q for _ in range(2)], lambda q: True))
    try:
        host = torch.zeros(256, dtype=torch.int32)
        device = torch.zeros(256, dtype=torch.int32)
        for into in (None, (host, device)):
            ctx = pack_step(entries, firsts, slots, tables, torch.device("cpu"), into=into)
            assert ctx.num_tokens == 9 and ctx.num_seqs == 4 and ctx.max_q_len == 5 and ctx.max_seq_len == 41 and not ctx.decode_only
            assert ctx.token_ids.tolist() == [7, 9, 3, 1, 4, 1, 5, 2, 6]
            assert ctx.positions.tolist() == [40, 3, 0, 1, 2, 3, 4, 17, 18]
            assert ctx.token_seq.tolist() == [0, 1, 2, 2, 2, 2, 2, 3, 3]
            assert ctx.seq_starts.tolist() == [0, 1, 2, 7, 9] and ctx.seq_lens.tolist() == [41, 4, 5, 19]
            assert ctx.first_positions.tolist() == firsts and ctx.state_slots.tolist() == slots
            assert ctx.want_rows.tolist() == [0, 6, 2, 8] and not ctx.wants_every_row_in_order
            assert [t.tolist() for t in ctx.block_tables] == tables
            assert ctx.plan("test_lengths_twice").tolist() == [[1, 1], [1, 1], [5, 5], [2, 2]] and ctx.plan("nobody registered this") is None
            assert ctx.host_q_lens == [1, 1, 5, 2] and ctx.request_ids == ["d0", "d1", "p0", "p1"]
        whole = pack_step([StepEntry("w", [1, 2, 3], [0, 1, 2])], [0], [0], [[[0]]], torch.device("cpu"))
        assert whole.wants_every_row_in_order and whole.want_rows.tolist() == [0, 1, 2]
        nothing_wanted = pack_step([StepEntry("w", [1, 2, 3], [])], [5], [0], [[[0]]], torch.device("cpu"))
        assert nothing_wanted.want_rows is None and nothing_wanted.positions.tolist() == [5, 6, 7]
    finally:
        unregister_step_plan("test_lengths_twice")
