"""Each kernel alone against its plain function (tests/plain_ops.py), at sizes other than the engine's."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_ops

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def _tol(dtype, scale=1.0):
    return (2e-6 if dtype == torch.float32 else 1.6e-2) * scale


@pytest.fixture(scope="module")
def ops():
    from tinyllama_inference_engine_b200 import ops as module

    assert torch.cuda.is_available(), "these tests need the GPU"
    module.core()
    return module


def _paged_case(rng, dtype, seq_lens, q_lens, kv_heads, head_dim, page_size, q_heads):
    """Random cache pages for requests of ``seq_lens`` tokens, the last ``q_lens`` of which are this step's rows."""
    num_pages = sum(-(-s // page_size) for s in seq_lens) + 3
    order = rng.permutation(num_pages)
    width = max(-(-s // page_size) for s in seq_lens) + 1
    table = -np.ones((len(seq_lens), width), dtype=np.int32)
    at = 0
    for i, s in enumerate(seq_lens):
        n = -(-s // page_size)
        table[i, :n] = order[at : at + n]
        at += n
    pages = (torch.randn(num_pages, 2, kv_heads, page_size, head_dim) * 0.5).to(dtype)
    positions, token_seq = [], []
    for i, (s, q) in enumerate(zip(seq_lens, q_lens)):
        positions += list(range(s - q, s))
        token_seq += [i] * q
    tokens = len(positions)
    qkv = (torch.randn(tokens, (q_heads + 2 * kv_heads) * head_dim) * 0.5).to(dtype)
    return qkv, pages, torch.tensor(positions, dtype=torch.int32), torch.tensor(token_seq, dtype=torch.int32), torch.from_numpy(table)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(ops, dtype):
    torch.manual_seed(0)
    table = torch.randn(131, 80).to(dtype)
    ids = torch.tensor([0, 130, 5, 5, 77], dtype=torch.int32)
    want = torch.empty(5, 80)
    plain_ops.embedding(table, ids, want)
    got = torch.empty(5, 80, device="cuda")
    ops.embedding(table.cuda(), ids.cuda(), got)
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,eps", [(80, 1e-4), (2048, 1e-5), (1000, 1e-6)])
def test_add_rmsnorm(ops, dtype, hidden, eps):
    torch.manual_seed(1)
    residual = torch.randn(7, hidden) * 3
    delta = torch.randn(7, hidden).to(dtype)
    weight = 1 + 0.1 * torch.randn(hidden)
    for use_delta, rows in ((True, None), (False, None), (False, torch.tensor([6, 0, 3], dtype=torch.int32))):
        r_plain, r_gpu = residual.clone(), residual.clone().cuda()
        n = 7 if rows is None else 3
        want = torch.empty(n, hidden, dtype=dtype)
        plain_ops.add_rmsnorm(r_plain, delta if use_delta else None, weight, eps, want, rows)
        got = torch.empty(n, hidden, dtype=dtype, device="cuda")
        ops.add_rmsnorm(r_gpu, delta.cuda() if use_delta else None, weight.cuda(), eps, got, None if rows is None else rows.cuda())
        assert torch.allclose(r_gpu.cpu(), r_plain, atol=1e-6)
        assert torch.allclose(got.cpu().float(), want.float(), atol=_tol(dtype, 8), rtol=_tol(dtype))


@pytest.mark.parametrize("hidden", [2048, 1000, 4096, 5120])
def test_add_rmsnorm_of_many_rows(ops, hidden):
    """Steps of hundreds of rows normalise with a warp per row (bfloat16 out; widths up to 4096, wider ones on the other kernel)."""
    torch.manual_seed(2)
    rows_total, eps = 300, 1e-5
    residual = torch.randn(rows_total, hidden) * 3
    delta = torch.randn(rows_total, hidden).bfloat16()
    weight = 1 + 0.1 * torch.randn(hidden)
    picked = torch.randperm(rows_total)[:260].to(torch.int32)
    for use_delta, rows in ((True, None), (False, None), (False, picked)):
        r_plain, r_gpu = residual.clone(), residual.clone().cuda()
        n = rows_total if rows is None else rows.shape[0]
        want = torch.empty(n, hidden, dtype=torch.bfloat16)
        plain_ops.add_rmsnorm(r_plain, delta if use_delta else None, weight, eps, want, rows)
        got = torch.full((n, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.add_rmsnorm(r_gpu, delta.cuda() if use_delta else None, weight.cuda(), eps, got, None if rows is None else rows.cuda())
        assert torch.allclose(r_gpu.cpu(), r_plain, atol=1e-6)
        assert torch.allclose(got.cpu().float(), want.float(), atol=_tol(torch.bfloat16, 8), rtol=_tol(torch.bfloat16))


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul_and_add(ops, dtype):
    torch.manual_seed(2)
    gate_up = (torch.randn(5, 2 * 176) * 2).to(dtype)
    want = torch.empty(5, 176, dtype=dtype)
    plain_ops.silu_mul(gate_up, want)
    got = torch.empty(5, 176, dtype=dtype, device="cuda")
    ops.silu_mul(gate_up.cuda(), got)
    assert torch.allclose(got.cpu().float(), want.float(), atol=_tol(dtype, 4), rtol=_tol(dtype))
    residual = torch.randn(5, 176)
    delta = torch.randn(5, 176).to(dtype)
    r = residual.clone().cuda()
    ops.add_(r, delta.cuda())
    assert torch.allclose(r.cpu(), residual + delta.float(), atol=1e-6)


@pytest.mark.parametrize("M,N,K", [(1, 256, 64), (37, 131, 80), (130, 70, 513), (3, 1000, 17)])
def test_gemm_fp32_is_true_32_bit(ops, M, N, K):
    torch.manual_seed(3)
    x, w = torch.randn(M, K), torch.randn(N, K)
    want = (x.double() @ w.double().T).float()
    got = torch.empty(M, N, device="cuda")
    ops.linear(x.cuda(), w.cuda(), got)
    # a reduced-precision (tf32 / bf16) product would be off by ~1e-3 * sqrt(K) here
    assert torch.allclose(got.cpu(), want, atol=2e-6 * K ** 0.5 * 4, rtol=1e-6)
    # one row alone gives bit-identical numbers: the order of a row's sum does not depend on the batch
    alone = torch.empty(1, N, device="cuda")
    ops.linear(x[M - 1 :].cuda(), w.cuda(), alone)
    assert torch.equal(alone[0], got[M - 1])


@pytest.mark.parametrize("M,N,K", [(1, 256, 64), (37, 136, 80), (130, 72, 520), (64, 2048, 2048)])
def test_linear_bf16(ops, M, N, K):
    torch.manual_seed(4)
    x, w = torch.randn(M, K).bfloat16(), torch.randn(N, K).bfloat16()
    want = x.float() @ w.float().T
    got = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ops.linear(x.cuda(), w.cuda(), got)
    assert torch.allclose(got.cpu().float(), want, atol=1e-2 * K ** 0.5, rtol=1e-2)
    got32 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    ops.linear(x.cuda(), w.cuda(), got32)
    assert torch.allclose(got32.cpu(), want, atol=2e-5 * K ** 0.5, rtol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_heads,kv_heads,head_dim,page_size,rotary_dim,theta", [(4, 2, 16, 16, 16, 1e4), (6, 2, 32, 32, 32, 5e5), (3, 3, 48, 16, 24, 777.0), (8, 1, 128, 64, 128, 1e4),
                                                                             (5, 1, 64, 16, 32, 1e4)])
def test_rope_store(ops, dtype, q_heads, kv_heads, head_dim, page_size, rotary_dim, theta):
    rng = np.random.default_rng(5)
    torch.manual_seed(5)
    seq_lens, q_lens = [4100, 17, page_size + 1, 1], [5, 17, 2, 1]
    qkv, pages, positions, token_seq, table = _paged_case(rng, dtype, seq_lens, q_lens, kv_heads, head_dim, page_size, q_heads)
    exponent = (np.float32(-2.0) * np.arange(rotary_dim // 2, dtype=np.float32)) / np.float32(rotary_dim)
    inv_freq = torch.from_numpy(np.power(np.float32(theta), exponent, dtype=np.float32))
    for write in (True, False):
        qkv_plain, pages_plain = qkv.clone(), pages.clone()
        plain_ops.rope_store(qkv_plain, positions, token_seq, table, inv_freq, rotary_dim, pages_plain, q_heads, kv_heads, head_dim, page_size, write)
        qkv_gpu, pages_gpu = qkv.clone().cuda(), pages.clone().cuda()
        ops.rope_store(qkv_gpu, positions.cuda(), token_seq.cuda(), table.cuda(), inv_freq.cuda(), rotary_dim, pages_gpu, q_heads, kv_heads, head_dim, page_size, write)
        q_width = q_heads * head_dim
        # position 4099 with 32-bit angles: sine and cosine of the two sides may differ in the last bits
        assert torch.allclose(qkv_gpu.cpu().float()[:, :q_width], qkv_plain.float()[:, :q_width], atol=_tol(dtype, 4) + 2e-4)
        assert torch.equal(qkv_gpu.cpu()[:, q_width:], qkv_plain[:, q_width:])
        assert torch.allclose(pages_gpu.cpu().float(), pages_plain.float(), atol=_tol(dtype, 4) + 2e-4)
        if not write:
            assert torch.equal(pages_gpu.cpu(), pages)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_heads,kv_heads,head_dim,page_size,window", [(4, 2, 16, 16, 0), (6, 2, 32, 32, 0), (3, 3, 48, 16, 0), (8, 1, 128, 64, 0), (4, 4, 80, 16, 0), (4, 2, 64, 16, 37), (32, 4, 64, 64, 0)])
def test_paged_attention(ops, dtype, q_heads, kv_heads, head_dim, page_size, window):
    rng = np.random.default_rng(6)
    torch.manual_seed(6)
    seq_lens = [300, page_size, page_size + 1, 1, 2 * page_size - 1, 131]
    q_lens = [7, page_size, 2, 1, 1, 131]
    qkv, pages, positions, token_seq, table = _paged_case(rng, dtype, seq_lens, q_lens, kv_heads, head_dim, page_size, q_heads)
    # one far key among hundreds: make a single early key of request 0 match its last query strongly
    q_row = sum(q_lens[:1]) - 1
    page, slot = int(table[0, 3 // page_size]), 3 % page_size
    for h in range(q_heads):
        qv = qkv.view(qkv.shape[0], -1, head_dim)[q_row, h].float()
        pages[page, 0, h // (q_heads // kv_heads), slot] = (qv * (6.0 / max(1e-3, float(qv.norm()) ** 2) * head_dim ** 0.5)).to(dtype)
    tokens = qkv.shape[0]
    want = torch.empty(tokens, q_heads * head_dim, dtype=dtype)
    plain_ops.paged_attention(qkv, pages, positions, token_seq, table, want, q_heads, kv_heads, head_dim, page_size, window)
    got = torch.empty(tokens, q_heads * head_dim, dtype=dtype, device="cuda")
    ops.paged_attention(qkv.cuda(), pages.cuda(), positions.cuda(), token_seq.cuda(), table.cuda(), got, q_heads, kv_heads, head_dim, page_size, window)
    assert torch.allclose(got.cpu().float(), want.float(), atol=_tol(dtype, 2) + (2e-6 if dtype == torch.float32 else 0)), float((got.cpu().float() - want.float()).abs().max())


def test_embedding_survives_an_id_outside_the_table_and_reports_it(ops):
    """An id the host never saw (a token sampled on the device from non-finite logits) must not be used as an address:
    row 0 is read instead and the device's error word says so; reading the word raises and clears it."""
    from tinyllama_inference_engine_b200.errors import KernelError

    table = torch.randn(50, 64).bfloat16().cuda()
    ids = torch.tensor([3, 50, -1, 0x7FFFFFFF, 49], dtype=torch.int32).cuda()
    got = torch.empty(5, 64, device="cuda")
    ops.check_device_errors(got.device)   # nothing is pending
    ops.embedding(table, ids, got)
    with pytest.raises(KernelError, match="outside the vocabulary"):
        ops.check_device_errors(got.device)
    ops.check_device_errors(got.device)   # cleared by the read that raised
    want = table.float()[[3, 0, 0, 0, 49]]
    assert torch.equal(got, want)


def test_sampling_non_finite_logits_still_gives_a_token_of_the_vocabulary(ops):
    vocab = 131
    logits = torch.randn(6, vocab)
    logits[0] = float("nan")
    logits[1] = float("-inf")
    logits[2, ::2] = float("nan")
    logits[3] = float("inf")
    logits[4, 5] = float("nan")
    cuda = lambda t: t.cuda()  # noqa: E731
    for temperature, top_p in ((0.0, 1.0), (0.9, 1.0), (0.9, 0.5)):
        out = torch.full((6,), -7, dtype=torch.int32, device="cuda")
        ops.sample(cuda(logits), cuda(torch.full((6,), temperature)), cuda(torch.full((6,), top_p)), cuda(torch.arange(6, dtype=torch.int64)),
                   cuda(torch.zeros(6, dtype=torch.int64)), out)
        tokens = out.cpu().tolist()
        assert all(0 <= t < vocab for t in tokens), (temperature, top_p, tokens)
    out = torch.full((6,), -7, dtype=torch.int32, device="cuda")
    ops.argmax(cuda(logits), out)
    assert all(0 <= t < vocab for t in out.cpu().tolist())


def test_argmax_and_sampling(ops):
    torch.manual_seed(7)
    logits = torch.randn(6, 1000)
    logits[0, 10] = logits[0, 700] = 9.0     # a tie: the lowest id wins
    logits[1, 999] = 12.0
    out = torch.empty(6, dtype=torch.int32, device="cuda")
    ops.argmax(logits.cuda(), out)
    want = torch.empty(6, dtype=torch.int32)
    plain_ops.argmax(logits, want)
    assert torch.equal(out.cpu(), want) and int(want[0]) == 10 and int(want[1]) == 999
    # rows long enough for several rounds of the 16-byte loads, maxima at a round's edge, at the end, and tied across rounds
    wide = torch.randn(4, 20000)
    wide[0, 4096 * 4 - 1] = 30.0
    wide[1, 19999] = 30.0
    wide[2, 17001] = wide[2, 4099] = 30.0
    wide[3, 0] = 30.0
    out = torch.empty(4, dtype=torch.int32, device="cuda")
    ops.argmax(wide.cuda(), out)
    assert out.cpu().tolist() == [4096 * 4 - 1, 19999, 4099, 0]
    greedy = torch.empty(4, dtype=torch.int32, device="cuda")
    ops.sample(wide.cuda(), torch.zeros(4).cuda(), torch.ones(4).cuda(), torch.zeros(4, dtype=torch.int64).cuda(), torch.zeros(4, dtype=torch.int64).cuda(), greedy)
    assert greedy.cpu().tolist() == [4096 * 4 - 1, 19999, 4099, 0]
    assert ops.uniform_from(11, 5) == plain_ops.uniform_from(11, 5) == pytest.approx(ops.core().tlie_uniform_from(11, 5))
    rows = 64
    logits = torch.randn(rows, 131) * 2
    temperature = torch.tensor([0.0, 0.8, 1.0, 1.5] * (rows // 4))
    top_p = torch.tensor([1.0, 1.0, 0.9, 0.5, 0.3, 1.0, 0.7, 0.95] * (rows // 8))
    seeds = torch.arange(rows, dtype=torch.int64) * 7 + 1
    counters = torch.arange(rows, dtype=torch.int64) % 5
    got = torch.empty(rows, dtype=torch.int32, device="cuda")
    ops.sample(logits.cuda(), temperature.cuda(), top_p.cuda(), seeds.cuda(), counters.cuda(), got)
    want = torch.empty(rows, dtype=torch.int32)
    plain_ops.sample(logits, temperature, top_p, seeds, counters, want)
    # the two sides sum probabilities in different orders: a draw that lands within rounding of a
    # boundary may fall on the neighbouring kept token, so demand near-total agreement, and exact for greedy rows
    agree = (got.cpu() == want)
    assert bool(agree[temperature == 0].all())
    assert int(agree.sum()) >= rows - 2, (got.cpu(), want)
    # the distribution: many draws of one row follow softmax(l / T) restricted by top_p
    row = torch.tensor([2.0, 1.0, 0.5, -1.0, -3.0] + [-20.0] * 45)
    n = 4096
    got = torch.empty(n, dtype=torch.int32, device="cuda")
    ops.sample(row.repeat(n, 1).cuda(), torch.full((n,), 0.7).cuda(), torch.full((n,), 0.8).cuda(), torch.full((n,), 3, dtype=torch.int64).cuda(), torch.arange(n, dtype=torch.int64).cuda(), got)
    p = torch.softmax(row / 0.7, 0)
    keep = p >= p[1]  # 0.8 is reached by the two most probable tokens
    expect = torch.where(keep, p, torch.zeros_like(p)) / p[keep].sum()
    freq = torch.bincount(got.cpu().long(), minlength=50).float() / n
    assert float((freq - expect).abs().max()) < 0.03


@pytest.mark.parametrize("q_heads,kv_heads,head_dim,page_size,window", [
    (32, 4, 64, 64, 0), (8, 8, 128, 64, 0), (32, 8, 128, 16, 0), (4, 2, 16, 16, 0), (6, 2, 32, 32, 0), (3, 3, 48, 16, 0),
    (16, 1, 64, 64, 0), (8, 2, 64, 32, 100), (10, 2, 80, 16, 33),
])
@pytest.mark.parametrize("splits", [1, 3, 16])
def test_decode_attention_split_kv(ops, q_heads, kv_heads, head_dim, page_size, window, splits):
    """The tensor-core decode kernel against the plain function: lengths at page and tile edges, one far key that dominates."""
    from tinyllama_inference_engine_b200.ops import fast

    rng = np.random.default_rng(8)
    torch.manual_seed(8)
    seq_lens = [1, 31, 32, 33, 64, 65, 127, 129, 700, 1153, 2 * page_size, 2 * page_size + 1]
    qkv, pages, positions, token_seq, table = _paged_case(rng, torch.bfloat16, seq_lens, [1] * len(seq_lens), kv_heads, head_dim, page_size, q_heads)
    for row in (8, 9):  # key 3 of the long requests matches every head's query strongly (only visible without a window)
        page, slot = int(table[row, 3 // page_size]), 3 % page_size
        for h in range(q_heads):
            qv = qkv.view(qkv.shape[0], -1, head_dim)[row, h].float()
            pages[page, 0, h // (q_heads // kv_heads), slot] = (qv * (6.0 * head_dim ** 0.5 / float(qv.norm()) ** 2)).bfloat16()
    want = torch.empty(len(seq_lens), q_heads * head_dim, dtype=torch.bfloat16)
    plain_ops.paged_attention(qkv, pages, positions, token_seq, table, want, q_heads, kv_heads, head_dim, page_size, window)
    got = torch.empty(len(seq_lens), q_heads * head_dim, dtype=torch.bfloat16, device="cuda")
    pages_gpu = pages.cuda()
    held = set(int(p) for p in table.flatten() if p >= 0)
    for page in range(pages.shape[0]):   # pages no request holds, and slots past a request's end: reading them would show
        if page not in held:
            pages_gpu[page] = float("nan")
    for i, n in enumerate(seq_lens):
        if n % page_size:
            pages_gpu[int(table[i, n // page_size]), :, :, n % page_size :] = float("nan")
    fast.decode_attention(qkv.cuda(), pages_gpu, positions.cuda(), table.cuda(), got, q_heads, kv_heads, head_dim, page_size, window, head_dim ** -0.5, splits)
    error = (got.cpu().float() - want.float()).abs().max(1).values
    assert float(error.max()) <= 1.6e-2 * 2, error


@pytest.mark.parametrize("q_heads,kv_heads,head_dim,page_size,window", [
    (32, 4, 64, 64, 0), (8, 8, 128, 64, 0), (4, 2, 16, 16, 0), (6, 2, 32, 32, 0), (3, 3, 48, 16, 0), (8, 2, 64, 32, 100), (10, 2, 80, 16, 33), (4, 1, 96, 16, 70),
])
def test_prefill_attention_flash(ops, q_heads, kv_heads, head_dim, page_size, window):
    """The tensor-core prompt kernel against the plain function: portions that start anywhere, tile and page edges, single rows."""
    from tinyllama_inference_engine_b200.ops import fast

    rng = np.random.default_rng(9)
    torch.manual_seed(9)
    seq_lens = [300, 64, 65, 1, 127, 131, 700, 2, 129]
    q_lens = [300, 64, 2, 1, 1, 131, 70, 2, 65]
    qkv, pages, positions, token_seq, table = _paged_case(rng, torch.bfloat16, seq_lens, q_lens, kv_heads, head_dim, page_size, q_heads)
    row = sum(q_lens[:6]) + 69  # the last row of the request of 700: key 5 far behind it dominates (if no window hides it)
    page, slot = int(table[6, 5 // page_size]), 5 % page_size
    for h in range(q_heads):
        qv = qkv.view(qkv.shape[0], -1, head_dim)[row, h].float()
        pages[page, 0, h // (q_heads // kv_heads), slot] = (qv * (6.0 * head_dim ** 0.5 / float(qv.norm()) ** 2)).bfloat16()
    tokens = qkv.shape[0]
    want = torch.empty(tokens, q_heads * head_dim, dtype=torch.bfloat16)
    plain_ops.paged_attention(qkv, pages, positions, token_seq, table, want, q_heads, kv_heads, head_dim, page_size, window)
    starts = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    firsts = np.array([s - q for s, q in zip(seq_lens, q_lens)], dtype=np.int32)
    from tinyllama_inference_engine_b200.ops.fast import ATTENTION_TILE_ROWS
    tiles = [[i, int(starts[i]) + off] for i, q in enumerate(q_lens) for off in range(0, q, ATTENTION_TILE_ROWS)]
    pages_gpu = pages.cuda()
    held = set(int(p) for p in table.flatten() if p >= 0)
    for page in range(pages.shape[0]):
        if page not in held:
            pages_gpu[page] = float("nan")
    for i, n in enumerate(seq_lens):
        if n % page_size:
            pages_gpu[int(table[i, n // page_size]), :, :, n % page_size :] = float("nan")
    got = torch.full((tokens, q_heads * head_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
    fast.prefill_attention(qkv.cuda(), pages_gpu, torch.tensor(tiles, dtype=torch.int32).cuda(), torch.from_numpy(starts).cuda(), torch.from_numpy(firsts).cuda(),
                           table.cuda(), got, q_heads, kv_heads, head_dim, page_size, window, head_dim ** -0.5)
    error = (got.cpu().float() - want.float()).abs().max(1).values
    assert float(error.max()) <= 1.6e-2 * 2, (int(error.argmax()), error.max())


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(130, 80), (2560, 2048), (2048, 5632), (1000, 200), (352, 176)])
def test_gemv_fused(ops, M, N, K):
    """The fused decode products: plain, with the norm in front, accumulating into the residual, and gated."""
    from tinyllama_inference_engine_b200.ops import fast

    torch.manual_seed(11)
    x = torch.randn(M, K).bfloat16()
    w = (torch.randn(N, K) * 0.05).bfloat16()
    want = x.float() @ w.float().T
    scale = float(want.abs().max())
    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 1.6e-2)):
        got = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
        fast.gemv_fused(x.cuda(), w.cuda(), got)
        assert torch.allclose(got.cpu().float(), want, atol=tol * scale, rtol=0)
    residual = torch.randn(M, N)
    got = residual.clone().cuda()
    fast.gemv_fused(x.cuda(), w.cuda(), got, epilogue="accumulate")
    assert torch.allclose(got.cpu(), residual + want, atol=1e-4 * scale + 1e-5)
    # long rows and few tiles take sixteen warps per CTA (K split sixteen ways): the same sums with the eight-warp kernel
    library = fast.gemv_library()
    library.tlie_gemv_set_wide_ctas(0)
    try:
        narrow = residual.clone().cuda()
        fast.gemv_fused(x.cuda(), w.cuda(), narrow, epilogue="accumulate")
    finally:
        library.tlie_gemv_set_wide_ctas(1)
    assert torch.allclose(narrow, got, atol=1e-4 * scale + 1e-5)
    # gated: silu of the first half of the rows times the second half, both rounded to bfloat16 first
    half = N // 2
    g, u = want[:, :half].bfloat16().float(), want[:, half:].bfloat16().float()
    gated = torch.empty(M, half, dtype=torch.bfloat16, device="cuda")
    fast.gemv_fused(x.cuda(), w.cuda(), gated, epilogue="gated")
    expect = (g / (1 + torch.exp(-g))) * u
    assert torch.allclose(gated.cpu().float(), expect, atol=1.6e-2 * float(expect.abs().max()) + 2e-3 * scale)
    # norm in front, with and without a gather of rows
    stream = torch.randn(M + 3, K) * 2
    norm_weight = 1 + 0.1 * torch.randn(K)
    for rows in (None, torch.randperm(M + 3)[:M].to(torch.int32)):
        normed = torch.empty(M, K, dtype=torch.bfloat16)
        plain_ops.add_rmsnorm(stream.clone(), None, norm_weight, 1e-5, normed, rows if rows is not None else torch.arange(M, dtype=torch.int32))
        want_n = normed.float() @ w.float().T
        got = torch.empty(M, N, dtype=torch.float32, device="cuda")
        fast.gemv_fused(stream.cuda(), w.cuda(), got, norm=(norm_weight.cuda(), 1e-5, None if rows is None else rows.cuda()))
        # the kernel rounds residual * weight to bfloat16 and scales the 32-bit sum: the same product, rounded elsewhere
        assert torch.allclose(got.cpu(), want_n, atol=6e-3 * float(want_n.abs().max())), float((got.cpu() - want_n).abs().max())
    # a product that completes the residual prepares the norm that follows: the next product reads what it left
    # (bfloat16(residual * weight) and the rows' sums of squares) and gives what the norm-in-front kernel gives
    if N % 8 == 0:
        residual = torch.randn(M, N) * 2
        next_weight = 1 + 0.1 * torch.randn(N)
        w2 = (torch.randn(40, N) * 0.05).bfloat16()
        total = residual.clone().cuda()
        x_out, squares = fast.prepared_norm_buffers(M, N, "cuda")
        fast.gemv_fused(x.cuda(), w.cuda(), total, epilogue="accumulate", prepare=(next_weight.cuda(), x_out, squares))
        assert torch.allclose(total.cpu(), residual + want, atol=1e-4 * scale + 1e-5)
        assert torch.equal(x_out.cpu(), (total.cpu() * next_weight).bfloat16())
        assert torch.allclose(squares.sum(1).cpu(), (total.cpu() ** 2).sum(1), rtol=1e-5)
        via_prepared = torch.empty(M, 40, dtype=torch.float32, device="cuda")
        fast.gemv_fused(x_out, w2.cuda(), via_prepared, prepared=(squares, 1e-5))
        via_norm = torch.empty(M, 40, dtype=torch.float32, device="cuda")
        fast.gemv_fused(total, w2.cuda(), via_norm, norm=(next_weight.cuda(), 1e-5, None))
        assert torch.allclose(via_prepared, via_norm, rtol=1e-5, atol=1e-6 * float(via_norm.abs().max()))


@pytest.mark.parametrize("M", [1, 17, 33, 64, 100, 127])
@pytest.mark.parametrize("N,K", [(130, 80), (2560, 2048), (2048, 5632), (1000, 200), (4096, 14336), (32000, 2048)])
def test_gemm_skinny(ops, M, N, K):
    """The weight-streaming tensor-core product of 17 to 127 rows against the 32-bit product: every epilogue, K cut over clusters of
    every size (the shapes give 1 to 8 parts), widths and depths that are no multiple of the tile, and the prepared-norm hand-over."""
    from tinyllama_inference_engine_b200.ops import fast

    torch.manual_seed(13)
    x = torch.randn(M, K).bfloat16()
    w = (torch.randn(N, K) * 0.05).bfloat16()
    want = x.float() @ w.float().T
    scale = float(want.abs().max())
    xc, wc = x.cuda(), w.cuda()
    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 1.6e-2)):
        got = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
        fast.gemm_skinny(xc, wc, got)
        error = (got.cpu().float() - want).abs()
        assert float(error.max()) <= tol * scale, (dtype, float(error.max()), scale, divmod(int(error.argmax()), N))
    residual = torch.randn(M, N)
    got = residual.clone().cuda()
    fast.gemm_skinny(xc, wc, got, epilogue="accumulate")
    assert torch.allclose(got.cpu(), residual + want, atol=1e-4 * scale + 1e-5)
    again = residual.clone().cuda()
    fast.gemm_skinny(xc, wc, again, epilogue="accumulate")
    assert torch.equal(again, got)   # the parts are added in rank order: the same bits every time
    half = N // 2
    g, u = want[:, :half].bfloat16().float(), want[:, half:2 * half].bfloat16().float()
    gated = torch.full((M, half), float("nan"), dtype=torch.bfloat16, device="cuda")
    fast.gemm_skinny(xc, wc[: 2 * half], gated, epilogue="gated")
    expect = (g / (1 + torch.exp(-g))) * u
    assert torch.allclose(gated.cpu().float(), expect, atol=1.6e-2 * float(expect.abs().max()) + 2e-3 * scale)
    # a product that completes the residual prepares the norm that follows; the next product scales its results by the rows' norms
    if N <= 4096:
        torch.manual_seed(14)
        residual = torch.randn(M, N) * 2
        next_weight = 1 + 0.1 * torch.randn(N)
        w2 = (torch.randn(72, N) * 0.05).bfloat16()
        total = residual.clone().cuda()
        x_out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        squares = torch.full((M, fast.skinny_square_runs(M, N, K) + 3), float("nan"), dtype=torch.float32, device="cuda")[:, :-3]   # rows may be strided
        fast.gemm_skinny(xc, wc, total, epilogue="accumulate", prepare=(next_weight.cuda(), x_out, squares))
        assert torch.allclose(total.cpu(), residual + want, atol=1e-4 * scale + 1e-5)
        assert torch.equal(x_out.cpu(), (total.cpu() * next_weight).bfloat16())
        assert torch.allclose(squares.sum(1).cpu(), (total.cpu() ** 2).sum(1), rtol=1e-5)
        if N % 8 == 0:
            normed = torch.empty(M, N, dtype=torch.bfloat16)
            plain_ops.add_rmsnorm(total.cpu().clone(), None, next_weight, 1e-5, normed)
            want_n = normed.float() @ w2.float().T
            via_prepared = torch.full((M, 72), float("nan"), dtype=torch.float32, device="cuda")
            fast.gemm_skinny(x_out, w2.cuda(), via_prepared, prepared=(squares, 1e-5))
            assert torch.allclose(via_prepared.cpu(), want_n, atol=6e-3 * float(want_n.abs().max())), float((via_prepared.cpu() - want_n).abs().max())
            gated_n = torch.full((M, 36), float("nan"), dtype=torch.bfloat16, device="cuda")
            fast.gemm_skinny(x_out, w2.cuda(), gated_n, epilogue="gated", prepared=(squares, 1e-5))
            gn, un = want_n[:, :36].bfloat16().float(), want_n[:, 36:].bfloat16().float()
            expect_n = (gn / (1 + torch.exp(-gn))) * un
            assert torch.allclose(gated_n.cpu().float(), expect_n, atol=2.5e-2 * float(expect_n.abs().max()) + 6e-3 * float(want_n.abs().max()))
    torch.cuda.synchronize()
    assert int(fast.tcgen05_error_flag(got.device)) == 0, "a bounded wait inside the kernel gave up"


@pytest.mark.parametrize("q_heads,kv_heads,head_dim,page_size,window,rotate", [
    (32, 4, 64, 64, 0, True), (8, 8, 128, 64, 0, True), (6, 2, 32, 32, 0, True), (8, 2, 64, 16, 100, True), (4, 2, 64, 16, 0, False), (12, 3, 96, 16, 0, True),
    (24, 2, 64, 16, 0, True),   # groups of twelve: the tile's upper rows are in use, four of them empty
])
@pytest.mark.parametrize("splits", [1, 5])
def test_decode_attention_with_rotation_and_cache_write(ops, q_heads, kv_heads, head_dim, page_size, window, rotate, splits):
    """The decode kernel doing rope_store's work itself: same output, same pages, as rope_store followed by attention."""
    from tinyllama_inference_engine_b200.ops import fast

    rng = np.random.default_rng(12)
    torch.manual_seed(12)
    seq_lens = [1, 32, 33, 64, 65, 700, 1153, 4097, 2 * page_size + 1]
    qkv, pages, positions, token_seq, table = _paged_case(rng, torch.bfloat16, seq_lens, [1] * len(seq_lens), kv_heads, head_dim, page_size, q_heads)
    inv_freq = None
    if rotate:
        exponent = (np.float32(-2.0) * np.arange(head_dim // 2, dtype=np.float32)) / np.float32(head_dim)
        inv_freq = torch.from_numpy(np.power(np.float32(10000.0), exponent, dtype=np.float32))
    for write in (True, False):
        qkv_plain, pages_plain = qkv.clone(), pages.clone()
        want = torch.empty(len(seq_lens), q_heads * head_dim, dtype=torch.bfloat16)
        plain_ops.attention_step(qkv_plain, positions, token_seq, table, inv_freq, head_dim if rotate else 0, pages_plain, want, q_heads, kv_heads, head_dim, page_size, window, None, write)
        pages_gpu = pages.clone().cuda()
        got = torch.empty(len(seq_lens), q_heads * head_dim, dtype=torch.bfloat16, device="cuda")
        fast.decode_attention(qkv.cuda(), pages_gpu, positions.cuda(), table.cuda(), got, q_heads, kv_heads, head_dim, page_size, window, head_dim ** -0.5, splits,
                              fuse_rope=True, inv_freq=None if inv_freq is None else inv_freq.cuda(), write_cache=write)
        assert float((got.cpu().float() - want.float()).abs().max()) <= 3.2e-2
        assert torch.allclose(pages_gpu.cpu().float(), pages_plain.float(), atol=1.6e-2 * 4 + 2e-4)
        if not write:
            assert torch.equal(pages_gpu.cpu(), pages)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 128), (2048, 2560, 2048), (300, 200, 136), (2048, 2048, 5632), (129, 1000, 2048), (1000, 131, 80),
                                   (4200, 2500, 72)])
@pytest.mark.parametrize("tile_n,pair", [(width, pair) for width in (128, 160, 192, 256) for pair in (False, True)] + [(288, False), (320, False), (288, True), (384, True), (480, True)])   # the wide tiles: two for single SMs, three for pairs
def test_gemm_tcgen05(ops, M, N, K, tile_n, pair):
    """The tcgen05 / TMA / tensor-memory product against a 32-bit product of the same bfloat16 values, tails included (the last
    shape gives every CTA several tiles at every width, the one-accumulator wide tile too)."""
    from tinyllama_inference_engine_b200.ops import fast

    torch.manual_seed(13)
    x = torch.randn(M, K).bfloat16()
    w = (torch.randn(N, K) * 0.05).bfloat16()
    want = x.float() @ w.float().T
    scale = float(want.abs().max())
    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 1.6e-2)):
        got = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
        fast.gemm_tcgen05(x.cuda(), w.cuda(), got, tile_n=tile_n, pair=pair)
        torch.cuda.synchronize()
        assert int(fast.tcgen05_error_flag(got.device)) == 0, "a bounded wait inside the kernel gave up"
        error = (got.cpu().float() - want).abs()
        assert float(error.max()) <= tol * scale, (float(error.max()), scale, int(error.argmax()) // N, int(error.argmax()) % N)


@pytest.mark.parametrize("pair,tile_n", [(False, 256), (True, 256), (True, 384), (True, 480)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (2048, 2048, 5632), (300, 200, 136), (1000, 132, 80), (129, 1000, 2048), (2100, 4100, 72)])
def test_gemm_tcgen05_accumulate(ops, M, N, K, pair, tile_n):
    """residual += product in the product's epilogue (bulk tensor reductions, each element once): twice in a row, tails included."""
    from tinyllama_inference_engine_b200.ops import fast

    torch.manual_seed(17)
    x = torch.randn(M, K).bfloat16()
    w = (torch.randn(N, K) * 0.05).bfloat16()
    start = torch.randn(M, N)
    product = x.float() @ w.float().T
    residual = start.clone().cuda()
    guard = torch.full((M + 1, N), 7.0, device="cuda")   # the rows behind the residual must stay as they are
    view = guard[:M]
    view.copy_(residual)
    for times in (1, 2):
        fast.gemm_tcgen05_accumulate(x.cuda(), w.cuda(), view, pair=pair, tile_n=tile_n)
        torch.cuda.synchronize()
        assert int(fast.tcgen05_error_flag(view.device)) == 0, "a bounded wait inside the kernel gave up"
        want = start + times * product
        error = (view.cpu() - want).abs()
        assert float(error.max()) <= 1e-4 * float(want.abs().max()), (times, float(error.max()), int(error.argmax()) // N, int(error.argmax()) % N)
        assert float((guard[M] - 7.0).abs().max()) == 0.0


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("M,inter,K", [(128, 128, 64), (2048, 5632, 2048), (300, 176, 136), (1000, 200, 80)])
def test_gemm_tcgen05_gated(ops, M, inter, K, pair):
    from tinyllama_inference_engine_b200.ops import fast

    torch.manual_seed(14)
    x = torch.randn(M, K).bfloat16()
    w = (torch.randn(2 * inter, K) * 0.05).bfloat16()
    both = (x.float() @ w.float().T).bfloat16().float()
    g, u = both[:, :inter], both[:, inter:]
    want = (g / (1 + torch.exp(-g))) * u
    got = torch.full((M, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    fast.gemm_tcgen05_gated(x.cuda(), w.cuda(), got, pair=pair)
    torch.cuda.synchronize()
    assert int(fast.tcgen05_error_flag(got.device)) == 0
    assert float((got.cpu().float() - want).abs().max()) <= 1.6e-2 * float(want.abs().max()) + 2e-3 * float(both.abs().max())


@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("q_heads,kv_heads,page_size,window", [(32, 4, 64, 0), (8, 2, 64, 100), (4, 4, 128, 0), (16, 1, 64, 37), (3, 3, 64, 0)])
def test_prefill_attention_tensor_memory(ops, q_heads, kv_heads, page_size, window, head_dim):
    """The tcgen05 prompt kernel (head size 64 and 128) against the plain function: portions that start anywhere, page edges, single rows."""
    from tinyllama_inference_engine_b200.ops.fast import paired_attention_tiles
    from tinyllama_inference_engine_b200.ops import fast

    rng = np.random.default_rng(15)
    torch.manual_seed(15)
    seq_lens = [300, 64, 65, 1, 127, 131, 700, 2, 129, 1000]
    q_lens = [300, 64, 2, 1, 1, 131, 70, 2, 65, 512]
    qkv, pages, positions, token_seq, table = _paged_case(rng, torch.bfloat16, seq_lens, q_lens, kv_heads, head_dim, page_size, q_heads)
    row = sum(q_lens[:6]) + 69
    page, slot = int(table[6, 5 // page_size]), 5 % page_size
    for h in range(q_heads):
        qv = qkv.view(qkv.shape[0], -1, head_dim)[row, h].float()
        pages[page, 0, h // (q_heads // kv_heads), slot] = (qv * (6.0 * head_dim ** 0.5 / float(qv.norm()) ** 2)).bfloat16()
    # A score far above everything before it, many key tiles into a row (request 9, position 588, key 568): the kernel keeps its
    # running output in tensor memory against a reference maximum and must rescale it there when the maximum jumps.
    late_row = sum(q_lens[:9]) + 100
    page, slot = int(table[9, 568 // page_size]), 568 % page_size
    for h in range(q_heads):
        qv = qkv.view(qkv.shape[0], -1, head_dim)[late_row, h].float()
        pages[page, 0, h // (q_heads // kv_heads), slot] = (qv * (16.0 * head_dim ** 0.5 / float(qv.norm()) ** 2)).bfloat16()
    tokens = qkv.shape[0]
    want = torch.empty(tokens, q_heads * head_dim, dtype=torch.bfloat16)
    plain_ops.paged_attention(qkv, pages, positions, token_seq, table, want, q_heads, kv_heads, head_dim, page_size, window)
    starts = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    firsts = np.array([s - q for s, q in zip(seq_lens, q_lens)], dtype=np.int32)
    tiles = paired_attention_tiles(q_lens, [int(f) for f in firsts], [int(x) for x in starts])
    assert len(tiles) // 4 == (sum(-(-q // 128) for q in q_lens) + 1) // 2
    pages_gpu = pages.cuda()
    held = set(int(p) for p in table.flatten() if p >= 0)
    for page in range(pages.shape[0]):
        if page not in held:
            pages_gpu[page] = float("nan")
    for i, n in enumerate(seq_lens):
        if n % page_size:
            pages_gpu[int(table[i, n // page_size]), :, :, n % page_size :] = float("nan")
    got = torch.full((tokens, q_heads * head_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
    fast.prefill_attention_tc(qkv.cuda(), pages_gpu, torch.tensor(tiles, dtype=torch.int32).view(-1, 4).cuda(), torch.from_numpy(starts).cuda(), torch.from_numpy(firsts).cuda(),
                              table.cuda(), got, q_heads, kv_heads, head_dim, page_size, window, head_dim ** -0.5)
    torch.cuda.synchronize()
    assert int(fast.tcgen05_error_flag(got.device)) == 0, "a bounded wait inside the kernel gave up"
    error = (got.cpu().float() - want.float()).abs().max(1).values
    assert float(error.max()) <= 1.6e-2 * 2, (int(error.argmax()), float(error.max()))


def test_hardware_probes_report_what_the_designs_rest_on():
    """The loops of csrc/probes.cu run to the end (every wait in them is bounded) and say what the kernels assume: a tensor-core
    product of 256 columns takes about twice one of 128, narrower ones cost no less than a floor, and a completed barrier is cheap."""
    from tinyllama_inference_engine_b200.ops.probes import hardware_probes

    report = hardware_probes("cuda:0")
    mma = report["mma_cycles"]
    wide, half, narrow = (mma[f"128 x {n} x 16, straight-line issue, one CTA per SM"] for n in (256, 128, 64))
    assert 100 < wide < 200 and 1.6 < wide / half < 2.4 and narrow <= half + 8
    assert mma["128 x 64 x 16, straight-line issue, two CTAs per SM"] > 1.5 * narrow       # two CTAs share one tensor core
    assert 0 < report["handoff_cycles"]["wait on a completed barrier"] < 400
    alone = report["arithmetic_cycles_per_64_values"]["64 exp2, one warp per scheduler"]
    shared = report["arithmetic_cycles_per_64_values"]["64 exp2, two warps per scheduler"]
    assert 400 < alone < 1200 and shared > 1.4 * alone                                       # the exponential unit is what two warps wait for


def test_product_comparison_runs_every_form(ops):
    """The committed comparison of the engine's products with the library's (kernel-bench --products) runs all forms at a small shape."""
    from tinyllama_inference_engine_b200.ops.probes import product_comparison

    report = product_comparison(256, 256, 512, 384, "cuda:0", launches=3)
    assert set(report) == {"qkv", "o", "gate_up", "down"}
    for line in report.values():
        assert line["own, one SM"] > 0 and line["own, SM pairs"] > 0 and any(key.startswith("library") and value > 0 for key, value in line.items())
        assert line["own_runs"] is False   # 256 rows: the library's


@pytest.mark.parametrize("M", [1, 8, 16])
def test_products_of_very_long_rows_stay_in_the_fused_kernel(ops, M):
    """K = 14,336 (the down projection of the 8B shapes): eight staged rows of x would not fit the kernel's shared memory, but with no
    more tiles than CTA slots nothing is staged at all, so the product and its residual add stay one kernel of this engine."""
    from tinyllama_inference_engine_b200.ops import fast

    torch.manual_seed(13)
    N, K = 4096, 14336
    x = torch.randn(M, K).bfloat16()
    w = (torch.randn(N, K) * 0.02).bfloat16()
    want = x.float() @ w.float().T
    scale = float(want.abs().max())
    residual = torch.randn(M, N)
    assert fast.gemv_fits(M, K, norm=False, N=N) and not fast.gemv_fits(M, K, norm=False)
    before = fast.library_gemm_calls
    got = residual.clone().cuda()
    ops.linear_accumulate(x.cuda(), w.cuda(), got)
    assert torch.allclose(got.cpu(), residual + want, atol=1e-4 * scale + 1e-5)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ops.linear(x.cuda(), w.cuda(), out)
    assert torch.allclose(out.cpu().float(), want, atol=1.6e-2 * scale, rtol=0)
    assert fast.library_gemm_calls == before
