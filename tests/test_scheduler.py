"""The scheduler's decisions and the cache manager's accounting, without a GPU."""
from __future__ import annotations

import random

import pytest
import torch

from tinyllama_inference_engine_b200.cache import CacheManager, PagePool
from tinyllama_inference_engine_b200.engine.request import FINISHED, Request, SamplingParams
from tinyllama_inference_engine_b200.engine.scheduler import Scheduler
from tinyllama_inference_engine_b200.errors import BatchError, EngineError, OutOfPages
from tinyllama_inference_engine_b200.parts.base import CacheNeed

FULL = CacheNeed("pages", kv_heads=2, head_dim=16)
WINDOW = CacheNeed("pages", kv_heads=2, head_dim=16, window=40)
STATE = CacheNeed("state", state_shape=(8,))


def test_page_pool_accounting():
    pool = PagePool(4)
    a = pool.allocate(3, "a")
    assert len(set(a)) == 3 and pool.free_count == 1
    with pytest.raises(OutOfPages):
        pool.allocate(2, "b")
    assert pool.free_count == 1  # nothing taken by the refused call
    with pytest.raises(EngineError, match="held by"):
        pool.free([a[0]], "b")
    pool.free([a[0]], "a")
    with pytest.raises(EngineError, match="freed twice"):
        pool.free([a[0]], "a")
    assert pool.allocate(1, "c") == [a[0]]  # the page freed last is used again first
    assert pool.reuses == 1
    pool.check()


def test_groups_have_pools_of_their_own_and_windows_give_pages_back():
    needs = {0: FULL, 1: WINDOW, 2: FULL, 3: STATE, 4: WINDOW}
    cache = CacheManager(needs, page_size=16, num_pages=12, max_requests=3, max_positions=192)
    assert [g.streams for g in cache.page_groups] == [[0, 2], [1, 4]]
    assert [g.streams for g in cache.state_groups] == [[3]]
    cache.admit("a")
    cache.reserve("a", 100)
    assert cache.free_pages() == [12 - 7, 12 - 7]
    cache.advance("a", 100)
    # window 40: queries at >= 100 read keys >= 61, so logical pages 0..2 (positions < 48) are passed
    assert cache.free_pages() == [5, 8]
    assert cache.records["a"].tables[1][:4] == [-1, -1, -1, cache.records["a"].tables[1][3]]
    cache.check()
    cache.reserve("a", 192)
    cache.advance("a", 192)
    assert cache.free_pages()[0] == 0 and cache.free_pages()[1] >= 8
    with pytest.raises(BatchError):
        cache.advance("a", 10)
    cache.release("a")
    assert cache.free_pages() == [12, 12]
    cache.check()


def test_a_page_may_hold_other_planes_than_keys_and_values():
    """What a page holds is the mixer's to say: one latent vector per token, or keys and values of different widths, are cache
    needs like any other; the manager gives them pools, tables and device memory without knowing what they mean."""
    latent = CacheNeed("pages", planes=((1, 24),))
    uneven = CacheNeed("pages", planes=((2, 16), (2, 48)), window=32)
    assert FULL.page_planes() == ((FULL.kv_heads, FULL.head_dim),) * 2 and FULL.uniform_planes()
    assert latent.uniform_planes() and not uneven.uniform_planes()
    cache = CacheManager({0: FULL, 1: latent, 2: uneven, 3: latent}, page_size=16, num_pages=6, max_requests=2, max_positions=96, device="cpu", poison_freed_pages=True)
    assert [g.streams for g in cache.page_groups] == [[0], [1, 3], [2]]
    assert tuple(cache.page_groups[1].tensor.shape) == (2, 6, 1, 1, 16, 24)
    assert [tuple(t.shape) for t in cache.page_groups[2].plane_tensors] == [(1, 6, 2, 16, 16), (1, 6, 2, 16, 48)]
    cache.admit("a")
    cache.reserve("a", 40)
    tables = torch.tensor(cache.block_table_rows(cache.page_groups[0], ["a"]), dtype=torch.int32)
    caches = cache.layer_caches([tables] * 3)
    assert tuple(caches[1].pages.shape) == (6, 1, 1, 16, 24) and caches[1].plane_pages == ()
    assert caches[2].pages is None and [tuple(t.shape) for t in caches[2].plane_pages] == [(6, 2, 16, 16), (6, 2, 16, 48)]
    expected = sum(t.numel() * 4 for g in cache.page_groups for t in g.tensors())
    assert cache.cache_bytes() == expected
    cache.release("a")
    cache.check()
    assert all(bool(torch.isnan(t).all()) for g in cache.page_groups for t in g.tensors())   # poisoned when given back


def test_reserve_is_all_or_nothing_across_groups():
    cache = CacheManager({0: FULL, 1: WINDOW}, page_size=16, num_pages=4, max_requests=2, max_positions=256)
    cache.admit("a")
    cache.reserve("a", 48)
    cache.advance("a", 48)
    cache.admit("b")
    before = cache.free_pages()
    with pytest.raises(OutOfPages):
        cache.reserve("b", 32)  # the full group has one page left, the window group has more
    assert cache.free_pages() == before and cache.records["b"].tables == {}
    with pytest.raises(OutOfPages, match="slots"):
        cache.admit("c")
    cache.check()


def test_random_orders_never_lose_or_double_a_page():
    rng = random.Random(0)
    cache = CacheManager({0: FULL, 1: WINDOW}, page_size=16, num_pages=24, max_requests=5, max_positions=400)
    live: dict[str, int] = {}
    made = 0
    for _ in range(3000):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            rid = f"r{made}"
            made += 1
            cache.admit(rid)
            live[rid] = 0
        elif action < 0.8 and live:
            rid = rng.choice(list(live))
            new_total = min(400, live[rid] + rng.choice([1, 1, 1, 2, 7, 16, 33]))
            try:
                cache.reserve(rid, new_total)
            except OutOfPages:
                victim = rng.choice(list(live))
                cache.release(victim)
                del live[victim]
            else:
                cache.advance(rid, new_total)
                live[rid] = new_total
        elif live:
            rid = rng.choice(list(live))
            cache.release(rid)
            del live[rid]
        cache.check()
        for rid, total in live.items():
            record = cache.records[rid]
            full, window = record.tables.get(0, []), record.tables.get(1, [])
            assert len(full) == len(window) == -(-total // 16)
            assert all(p >= 0 for p in full)
            first_needed = max(0, total - 40 + 1) // 16
            assert all((p < 0) == (i < first_needed) for i, p in enumerate(window))
    for rid in list(live):
        cache.release(rid)
    assert cache.free_pages() == [24, 24]
    assert all(g.pool.reuses > 0 for g in cache.page_groups)


def _scheduler(num_pages=8, budget=32, max_requests=4, max_positions=512):
    cache = CacheManager({0: FULL}, page_size=16, num_pages=num_pages, max_requests=max_requests, max_positions=max_positions)
    return Scheduler(cache, budget, max_requests, max_positions), cache


def _run(scheduler, cache, portions):
    """What the engine does after schedule(): reserve, advance, and pretend a token was sampled."""
    for p in portions:
        r = p.request
        if not cache.has(r.request_id):
            cache.admit(r.request_id)
        cache.reserve(r.request_id, r.computed + p.num_tokens)
        cache.advance(r.request_id, r.computed + p.num_tokens)
        samples = p.samples
        r.computed += p.num_tokens
        if samples:
            r.generated.append(7)
            if len(r.generated) >= r.params.max_tokens:
                scheduler.finish(r, "length")
    cache.check()


def test_budget_cuts_prompts_and_decodes_go_first():
    s, cache = _scheduler(num_pages=32, budget=32)
    a = Request("a", list(range(50)), SamplingParams(max_tokens=4))
    b = Request("b", list(range(20)), SamplingParams(max_tokens=4))
    s.add(a)
    s.add(b)
    first = s.schedule()
    assert [(p.request.request_id, p.num_tokens, p.samples) for p in first] == [("a", 32, False)]
    _run(s, cache, first)
    second = s.schedule()
    assert [(p.request.request_id, p.num_tokens, p.samples) for p in second] == [("a", 18, True), ("b", 14, False)]
    _run(s, cache, second)
    third = s.schedule()
    # a decodes (one token) before b's prompt goes on
    assert [(p.request.request_id, p.num_tokens, p.samples) for p in third] == [("a", 1, True), ("b", 6, True)]
    _run(s, cache, third)
    while s.has_unfinished():
        _run(s, cache, s.schedule())
    assert a.state == b.state == FINISHED and len(a.generated) == len(b.generated) == 4
    assert cache.free_pages() == [32] and not cache.records


def test_rotating_cursor_serves_every_decode():
    s, cache = _scheduler(num_pages=64, budget=8, max_requests=4)
    requests = [Request(f"r{i}", [1], SamplingParams(max_tokens=30)) for i in range(4)]
    for r in requests:
        s.add(r)
    _run(s, cache, s.schedule())
    assert len(s.running) == 4
    s.max_batch_tokens = 2  # from now on only two of the four decodes fit a step
    served = {r.request_id: 0 for r in requests}
    for _ in range(8):
        portions = s.schedule()
        assert len(portions) == 2
        for p in portions:
            served[p.request.request_id] += 1
        _run(s, cache, portions)
    assert set(served.values()) == {4}


def test_requests_are_refused_at_submission_when_they_cannot_fit():
    s, _ = _scheduler(num_pages=4, max_positions=128)
    with pytest.raises(EngineError, match="context length"):
        s.add(Request("x", [1] * 120, SamplingParams(max_tokens=9)))
    with pytest.raises(EngineError, match="even alone"):
        s.add(Request("y", [1] * 60, SamplingParams(max_tokens=10)))
    s.add(Request("z", [1] * 60, SamplingParams(max_tokens=5)))  # 64 positions cached at most: exactly 4 pages


def test_when_pages_run_out_the_newest_request_is_preempted_and_recomputes():
    s, cache = _scheduler(num_pages=6, budget=64, max_requests=4, max_positions=96)
    a = Request("a", [1] * 30, SamplingParams(max_tokens=40))
    b = Request("b", [2] * 30, SamplingParams(max_tokens=40))
    s.add(a)
    s.add(b)
    steps = 0
    saw_preempted_state = False
    while s.has_unfinished():
        portions = s.schedule()
        assert portions
        saw_preempted_state |= b.preemptions > 0 and b.computed == 0 and b in s.waiting
        _run(s, cache, portions)
        steps += 1
        assert steps < 500
    # both need ceil(69/16) = 5 pages at the end, the pool has 6: b (admitted last) had to give way
    assert s.preemptions >= 1 and b.preemptions >= 1 and a.preemptions == 0 and saw_preempted_state
    assert len(a.generated) == len(b.generated) == 40
    assert cache.free_pages() == [6] and not cache.records


def test_a_new_request_never_preempts_a_running_one():
    s, cache = _scheduler(num_pages=4, budget=64, max_positions=128)
    a = Request("a", [1] * 40, SamplingParams(max_tokens=8))
    s.add(a)
    _run(s, cache, s.schedule())
    b = Request("b", [1] * 40, SamplingParams(max_tokens=8))
    s.add(b)
    portions = s.schedule()
    assert [p.request.request_id for p in portions] == ["a"] and s.preemptions == 0 and b in s.waiting
    while s.has_unfinished():
        _run(s, cache, s.schedule())
    assert s.preemptions == 0 and len(b.generated) == 8


def test_random_workloads_finish_with_exact_counts_and_no_leak():
    rng = random.Random(1)
    for trial in range(20):
        s, cache = _scheduler(num_pages=rng.choice([6, 9, 16]), budget=rng.choice([8, 24, 64]), max_requests=rng.choice([2, 4]), max_positions=96)
        requests = []
        for i in range(rng.randint(1, 9)):
            r = Request(f"r{i}", [1] * rng.randint(1, 50), SamplingParams(max_tokens=rng.randint(1, 40)))
            s.add(r)
            requests.append(r)
        steps = 0
        while s.has_unfinished():
            portions = s.schedule()
            assert sum(p.num_tokens for p in portions) <= s.max_batch_tokens
            assert len({p.request.request_id for p in portions}) == len(portions)
            _run(s, cache, portions)
            steps += 1
            assert steps < 5000
        assert all(r.state == FINISHED and len(r.generated) == r.params.max_tokens for r in requests)
        assert cache.free_pages() == cache.total_pages() and not cache.records
