"""Host wrappers of the engine's CUDA kernels.

Every function here launches a hand-written sm_100a kernel on the current CUDA
stream.  There is no CPU fallback and no library model code behind them: tensors
must live on a CUDA device, and a missing compiler or a failed build raises
``KernelError``.  Matrix products of the bfloat16 path may go to the vendor library
(as the reference's do, src/cuda/kernels.cu:342-368) until the engine's own
tensor-core kernel covers the shape; the 32-bit path always uses the engine's own
32-bit product.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..errors import KernelError
from .build import build_library, load_library

CORE_SOURCES = ["elementwise.cu", "rope_cache.cu", "attention_generic.cu", "gemm_fp32.cu", "sampling.cu"]
_F32, _BF16 = 0, 1
launch_count = 0  # kernels of this engine launched by this process (a claim the bench reports)


def core():
    lib = load_library("tlie_core", CORE_SOURCES)
    if not getattr(lib, "_tlie_typed", False):
        lib.tlie_uniform_from.restype = c_float
        lib.tlie_uniform_from.argtypes = [c_longlong, c_longlong]
        lib._tlie_typed = True
    return lib


def build_all() -> list:
    """Compile every kernel set (used by the build check); returns the library paths."""
    return [build_library("tlie_core", CORE_SOURCES)] + fast.build_all()


def _code(tensor: torch.Tensor) -> int:
    if tensor.dtype == torch.float32:
        return _F32
    if tensor.dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {tensor.dtype}", code="invalid_dtype")


def _ptr(tensor: torch.Tensor | None) -> c_void_p:
    if tensor is None:
        return c_void_p(0)
    if not tensor.is_cuda:
        raise KernelError("this engine has no CPU path: a kernel was given a tensor that is not on a CUDA device")
    if not tensor.is_contiguous():
        raise KernelError("kernels take contiguous tensors")
    return c_void_p(tensor.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> c_void_p:
    """The handle of torch's current stream on the current device.

    Every kernel launch asks for it; ``torch.cuda.current_stream()`` builds a Stream object each time (several microseconds, a
    fifth of the host time of a short prompt step), the two calls used here only read the handle."""
    if _raw_stream is not None and _device_index is not None:
        return c_void_p(_raw_stream(_device_index()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(status: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if status != 0:
        raise KernelError(f"{what} failed to launch: CUDA error {status}")


def _i32(tensor: torch.Tensor | None, what: str) -> c_void_p:
    if tensor is not None and tensor.dtype != torch.int32:
        raise KernelError(f"{what} must be int32, got {tensor.dtype}", code="invalid_dtype")
    return _ptr(tensor)


# --- the device's error word -------------------------------------------------------------
# Kernels that can notice a fault without a host in the loop record it in one int32 per device: bit 0, a bounded wait
# inside a tensor-core kernel gave up (its results are garbage); bit 1, a token id outside the vocabulary reached the
# embedding (row 0 was read instead).  The engine reads the word wherever it synchronises with the device anyway.
_error_flags: dict[torch.device, torch.Tensor] = {}
DEVICE_ERRORS = {1: "a bounded wait inside a tensor-core kernel gave up; the step's results are not valid",
                 2: "a token id outside the vocabulary reached the embedding kernel (non-finite logits upstream?)"}


def error_flag(device: torch.device) -> torch.Tensor:
    """The device's error word (int32 [1]); kernels set bits in it, ``raise_for_error_word`` names and clears them."""
    device = torch.device(device)
    if device not in _error_flags:
        _error_flags[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[device]


def raise_for_error_word(word: int, device: torch.device) -> None:
    """Raise KernelError if ``word`` (a host copy of the device's error word) has a bit set, clearing the word on the device."""
    if word:
        error_flag(device).zero_()
        reasons = [text for bit, text in DEVICE_ERRORS.items() if word & bit] or [f"unknown error bits {word:#x}"]
        raise KernelError("the device reported: " + "; ".join(reasons))


def check_device_errors(device: torch.device) -> None:
    """Read the device's error word (this synchronises) and raise if a kernel reported a fault."""
    device = torch.device(device)
    if device in _error_flags:
        raise_for_error_word(int(_error_flags[device].item()), device)


# --- rows --------------------------------------------------------------------------------
def embedding(table: torch.Tensor, ids: torch.Tensor, residual: torch.Tensor) -> None:
    """residual[t] = float(table[ids[t]]); an id outside the table reads row 0 and sets bit 1 of the device's error word."""
    rows, hidden = residual.shape
    if table.shape[1] != hidden:
        raise KernelError("embedding: the table's width is not the residual's", code="invalid_shape")
    _check(core().tlie_embedding(_code(table), _ptr(table), _i32(ids, "ids"), _ptr(residual), c_int(rows), c_int(hidden), c_int(table.shape[0]),
                                 _ptr(error_flag(residual.device)), _stream()), "embedding")


def add_rmsnorm(residual, delta, weight, eps: float, out, rows=None) -> None:
    """Optional ``residual += delta`` in 32-bit, then ``out = rmsnorm(residual) * weight``.

    With ``rows`` (int32) only those rows are normalised (and ``delta`` must be None).
    """
    if residual.dtype != torch.float32 or weight.dtype != torch.float32:
        raise KernelError("the residual stream and norm weights are 32-bit", code="invalid_dtype")
    if rows is not None and delta is not None:
        raise KernelError("add_rmsnorm cannot add a delta while gathering rows")
    out_rows, hidden = out.shape
    if weight.numel() != hidden or residual.shape[1] != hidden:
        raise KernelError("add_rmsnorm: widths differ", code="invalid_shape")
    if delta is not None and (delta.shape != residual.shape or delta.dtype != out.dtype):
        raise KernelError("add_rmsnorm: delta must match the residual's shape and the output's dtype", code="invalid_shape")
    _check(
        core().tlie_add_rmsnorm(_code(out), _ptr(residual), _ptr(delta), _i32(rows, "rows"), _ptr(weight), c_float(eps), _ptr(out), c_int(out_rows), c_int(hidden), _stream()),
        "add_rmsnorm",
    )


def add_(residual, delta) -> None:
    _check(core().tlie_add(_code(delta), _ptr(residual), _ptr(delta), c_longlong(residual.numel()), _stream()), "add")


def silu_mul(gate_up, out) -> None:
    rows, inter = out.shape
    if gate_up.shape != (rows, 2 * inter) or gate_up.dtype != out.dtype:
        raise KernelError("silu_mul: gate_up must be [rows, 2 * inter] of the output's dtype", code="invalid_shape")
    _check(core().tlie_silu_mul(_code(out), _ptr(gate_up), _ptr(out), c_int(rows), c_int(inter), _stream()), "silu_mul")


# --- matrix products --------------------------------------------------------------------
def linear(x, weight, out) -> None:
    """out[M, N] = x[M, K] . weight[N, K]^T in the tensors' dtype (32-bit accumulation)."""
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"linear: shapes {tuple(x.shape)} x {tuple(weight.shape)}^T -> {tuple(out.shape)} do not fit", code="invalid_shape")
    if x.dtype == torch.float32:
        if weight.dtype != torch.float32 or out.dtype != torch.float32:
            raise KernelError("linear: the 32-bit path takes 32-bit weights and outputs", code="invalid_dtype")
        _check(core().tlie_gemm_nt_f32(_ptr(x), _ptr(weight), _ptr(out), c_int(M), c_int(N), c_int(K), _stream()), "gemm_nt_f32")
        return
    fast.linear_bf16(x, weight, out)


def fused_rows_limit(dtype: torch.dtype, device: torch.device) -> int:
    """Up to how many rows a step may use the fused decode kernels (0: never, as in the 32-bit path)."""
    if dtype != torch.bfloat16 or device.type != "cuda":
        return 0
    return fast.FUSED_MAX_ROWS


# A product that completes the residual leaves the next norm's input for the product after it, from this many rows on
# (measured per decode step of the 1.1B shapes: 2 % slower with 1 or 2 rows, 2 to 3 % faster with 4 to 8).
use_prepared_norms = True
PREPARED_NORM_MIN_ROWS = 3


class LazyNorm:
    """A normalised activation that is not computed yet: rmsnorm(residual[rows]) * weight.

    A product that can apply the norm while it loads its operand takes this in the place of a tensor
    (``norm_linear``); anything else calls ``tensor()``.  ``prepared``: set by the product that completed the residual
    (``linear_accumulate(..., prepare=this)``) to (bfloat16(residual * weight), sums of squares per 16 columns), which
    ``norm_linear`` then reads instead of working them out again in every thread block.
    """

    def __init__(self, residual, weight, eps: float, rows, materialize):
        self.residual, self.weight, self.eps, self.rows = residual, weight, eps, rows
        self._materialize = materialize
        self.shape = (residual.shape[0] if rows is None else rows.shape[0], residual.shape[1])
        self.prepared = None
        self.buffers = None    # where ``prepared`` is to be written (buffers of fixed address), or None for fresh ones

    def tensor(self):
        return self._materialize()


def norm_linear(x: "LazyNorm", weight, out, gated: bool = False) -> None:
    """out = rmsnorm(residual) * norm_weight . weight^T in one kernel (``gated``: silu(gate) * up of the two halves)."""
    epilogue = "gated" if gated else "store"
    if fast.gemv_fits(out.shape[0], weight.shape[1], norm=True, gated=gated):
        if x.prepared is not None:
            fast.gemv_fused(x.prepared[0], weight, out, prepared=(x.prepared[1], x.eps), epilogue=epilogue)
        else:
            fast.gemv_fused(x.residual, weight, out, norm=(x.weight, x.eps, x.rows), epilogue=epilogue)
    elif fast.use_skinny and x.prepared is not None and fast.skinny_fits(out.shape[0], weight, x.prepared[0]) and out.is_contiguous():
        # the rows' scale is applied to the product's result: the operand is bfloat16(residual * norm weight) as it was left
        fast.gemm_skinny(x.prepared[0], weight, out, epilogue=epilogue, prepared=(x.prepared[1], x.eps))
    elif gated:
        linear_gated(x.tensor(), weight, out)
    else:
        linear(x.tensor(), weight, out)


def can_accumulate(rows: int, weight) -> bool:
    """Whether ``linear_accumulate`` is one kernel for a step of this many rows beyond the fused row limit."""
    return fast.can_accumulate(rows, weight)


def linear_accumulate(x, weight, residual, prepare: "LazyNorm | None" = None) -> None:
    """residual += x . weight^T, the sum in 32-bit, in one kernel (bfloat16 x; up to 16 rows in the register-fed weight-streaming
    kernel, up to 127 in the tensor-core one, for prompt portions in the tensor-core product's epilogue).

    ``prepare``: the lazy norm of this residual (all rows) that the next product will consume; the kernel then leaves that
    norm's input beside the residual (``prepare.prepared``), written by the threads that hold the finished sums."""
    rows = x.shape[0]
    preparing = (prepare is not None and prepare.rows is None and prepare.residual is residual and use_prepared_norms
                 and residual.shape[0] >= PREPARED_NORM_MIN_ROWS)
    if fast.gemv_fits(rows, weight.shape[1], norm=False, N=weight.shape[0]):
        if preparing:
            buffers = fast.prepared_norm_buffers(residual.shape[0], residual.shape[1], residual.device) if prepare.buffers is None else prepare.buffers
            fast.gemv_fused(x, weight, residual, epilogue="accumulate", prepare=(prepare.weight, buffers[0], buffers[1]))
            prepare.prepared = buffers
        else:
            fast.gemv_fused(x, weight, residual, epilogue="accumulate")
    elif fast.use_skinny and fast.skinny_fits(rows, weight, x) and residual.is_contiguous():
        buffers = None
        if preparing:
            buffers = fast.prepared_norm_buffers(residual.shape[0], residual.shape[1], residual.device) if prepare.buffers is None else prepare.buffers
            runs = fast.skinny_square_runs(rows, weight.shape[0], weight.shape[1])   # this kernel's partial sums per row: one per CTA that finishes a run of columns
            if runs > buffers[1].shape[1]:
                buffers = None   # a narrow matrix cut many ways: more partial sums than the buffer has room for
        if buffers is not None:
            squares = buffers[1][:, :runs]
            fast.gemm_skinny(x, weight, residual, epilogue="accumulate", prepare=(prepare.weight, buffers[0], squares))
            prepare.prepared = (buffers[0], squares)
        else:
            fast.gemm_skinny(x, weight, residual, epilogue="accumulate")
    elif x.dtype == torch.bfloat16 and fast.can_accumulate(rows, weight) and x.is_contiguous() and residual.is_contiguous():
        fast.gemm_tcgen05_accumulate(x, weight, residual)
    else:
        delta = torch.empty((rows, weight.shape[0]), dtype=x.dtype, device=x.device)
        linear(x, weight, delta)
        add_(residual, delta)


def linear_gated(x, weight, out) -> None:
    """out = silu(x . gate^T) * (x . up^T) for weight = [gate rows | up rows], in one kernel."""
    if fast.gemv_fits(x.shape[0], weight.shape[1], norm=False, gated=True):
        fast.gemv_fused(x, weight, out, epilogue="gated")
    elif fast.use_tcgen05 and fast.gated_takes(x.shape[0], weight.shape[0], weight.shape[1]) and weight.shape[1] % 8 == 0 and x.is_contiguous():
        fast.gemm_tcgen05_gated(x, weight, out)
    elif fast.use_skinny and fast.skinny_fits(x.shape[0], weight, x) and out.is_contiguous() and out.dtype == torch.bfloat16:
        fast.gemm_skinny(x, weight, out, epilogue="gated")
    else:
        gate_up = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)
        linear(x, weight, gate_up)
        silu_mul(gate_up, out)


# --- position encoding and cache write ---------------------------------------------------
def rope_store(qkv, positions, token_seq, block_table, inv_freq, rotary_dim: int, pages, q_heads: int, kv_heads: int, head_dim: int, page_size: int, write_cache: bool = True) -> None:
    """Rotate q (in place) and k, and store k, v of every token into its request's pages."""
    tokens = qkv.shape[0]
    if qkv.shape[1] != (q_heads + 2 * kv_heads) * head_dim:
        raise KernelError("rope_store: qkv width does not fit the head counts", code="invalid_shape")
    if write_cache and pages.dtype != qkv.dtype:
        raise KernelError("rope_store: pages and qkv differ in dtype", code="invalid_dtype")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("rope_store: inv_freq must hold rotary_dim / 2 32-bit frequencies", code="invalid_shape")
    _check(
        core().tlie_rope_store(
            _code(qkv), _ptr(qkv), _i32(positions, "positions"), _i32(token_seq, "token_seq"), _i32(block_table, "block_table"),
            c_int(block_table.shape[1]), _ptr(inv_freq), c_int(rotary_dim if inv_freq is not None else 0), _ptr(pages if write_cache else None),
            c_int(tokens), c_int(q_heads), c_int(kv_heads), c_int(head_dim), c_int(page_size), c_int(1 if write_cache else 0), _stream(),
        ),
        "rope_store",
    )


# --- attention -----------------------------------------------------------------------------
def paged_attention(qkv, pages, positions, token_seq, block_table, out, q_heads: int, kv_heads: int, head_dim: int, page_size: int, window: int = 0, scale: float | None = None, batch=None) -> None:
    """Attention of every query row over its request's cached keys up to its own position.

    ``qkv`` rows start with the (already rotated) q heads; ``batch`` may carry the
    step's shape so that a faster kernel can be chosen for bfloat16.
    """
    tokens = qkv.shape[0]
    if head_dim % 16 != 0 or head_dim > 256:
        raise KernelError(f"attention kernels take head sizes that are multiples of 16 up to 256, got {head_dim}", code="invalid_shape")
    if q_heads % kv_heads != 0:
        raise KernelError("attention: query heads must be a multiple of key/value heads", code="invalid_shape")
    if scale is None:
        scale = head_dim ** -0.5
    if qkv.dtype == torch.bfloat16:
        if fast.paged_attention_bf16(qkv, pages, positions, token_seq, block_table, out, q_heads, kv_heads, head_dim, page_size, window, scale, batch):
            return
    _check(
        core().tlie_paged_attention_generic(
            _code(qkv), _ptr(qkv), c_int(qkv.shape[1]), _ptr(pages), _i32(positions, "positions"), _i32(token_seq, "token_seq"),
            _i32(block_table, "block_table"), c_int(block_table.shape[1]), _ptr(out), c_int(tokens), c_int(q_heads), c_int(kv_heads),
            c_int(head_dim), c_int(page_size), c_int(window), c_float(scale), _stream(),
        ),
        "paged_attention_generic",
    )


def attention_step(qkv, positions, token_seq, block_table, inv_freq, rotary_dim: int, pages, out, q_heads: int, kv_heads: int,
                   head_dim: int, page_size: int, window: int = 0, scale: float | None = None, write_cache: bool = True, batch=None) -> None:
    """Rotate q and k, store k and v in the pages, and attend: ``rope_store`` then ``paged_attention``, in one kernel where one exists."""
    if qkv.dtype == torch.bfloat16:
        if fast.can_fuse_rope_into_decode(batch, qkv, head_dim, q_heads, kv_heads, inv_freq, rotary_dim):
            splits = fast.decode_splits(batch.num_seqs, kv_heads, batch.max_seq_len)
            fast.decode_attention(qkv, pages, positions, block_table, out, q_heads, kv_heads, head_dim, page_size, window,
                                  head_dim ** -0.5 if scale is None else scale, splits, fuse_rope=True, inv_freq=inv_freq, write_cache=write_cache)
            return
    rope_store(qkv, positions, token_seq, block_table, inv_freq, rotary_dim, pages, q_heads, kv_heads, head_dim, page_size, write_cache)
    paged_attention(qkv, pages, positions, token_seq, block_table, out, q_heads, kv_heads, head_dim, page_size, window, scale, batch)


# --- sampling ------------------------------------------------------------------------------
def argmax(logits, out) -> None:
    """out[r] = index of the largest logit of row r, the lowest index on ties."""
    if logits.dtype != torch.float32:
        raise KernelError("sampling takes 32-bit logits", code="invalid_dtype")
    _check(core().tlie_argmax(_ptr(logits), c_int(logits.shape[0]), c_int(logits.shape[1]), _i32(out, "out"), _stream()), "argmax")


def sample(logits, temperature, top_p, seeds, counters, out) -> None:
    """Temperature / top-p sampling per row; rows with temperature <= 0 are greedy."""
    if logits.dtype != torch.float32 or temperature.dtype != torch.float32 or top_p.dtype != torch.float32:
        raise KernelError("sampling takes 32-bit logits, temperatures and top_p", code="invalid_dtype")
    if seeds.dtype != torch.int64 or counters.dtype != torch.int64:
        raise KernelError("sampling takes int64 seeds and counters", code="invalid_dtype")
    _check(
        core().tlie_sample(_ptr(logits), c_int(logits.shape[0]), c_int(logits.shape[1]), _ptr(temperature), _ptr(top_p), _ptr(seeds), _ptr(counters), _i32(out, "out"), _stream()),
        "sample",
    )


def decode_advance(token_ids, sampled, positions, seq_lens, first_positions, counters, mailbox=None, steps_done=None) -> None:
    """token_ids = sampled; positions, seq_lens, first_positions and counters move on by one.

    ``mailbox``: a pinned host int32 tensor of ``count + 2`` words that the kernel writes over the bus (the tokens, the device error
    word, then the number of the step from the device counter ``steps_done``), so that the host can poll for the step's result."""
    count = token_ids.shape[0]
    box, flag, done = c_void_p(0), c_void_p(0), c_void_p(0)
    if mailbox is not None:
        if mailbox.dtype != torch.int32 or not mailbox.is_pinned() or mailbox.numel() < count + 2 or steps_done is None or steps_done.dtype != torch.int32:
            raise KernelError("decode_advance: the mailbox is pinned host int32 of count + 2 words, with a device int32 step counter", code="invalid_shape")
        box, flag, done = c_void_p(mailbox.data_ptr()), _ptr(error_flag(token_ids.device)), _ptr(steps_done)
    _check(
        core().tlie_decode_advance(_i32(token_ids, "token_ids"), _i32(sampled, "sampled"), _i32(positions, "positions"), _i32(seq_lens, "seq_lens"),
                                   _i32(first_positions, "first_positions"), _ptr(counters), c_int(count), box, flag, done, _stream()),
        "decode_advance",
    )


def uniform_from(seed: int, counter: int) -> float:
    """The uniform number in [0, 1) that draw ``counter`` of a request with ``seed`` uses."""
    mask = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + (counter + 1) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return (z >> 40) / 16777216.0


from . import fast  # noqa: E402  (the bfloat16 kernels; at the end because it refers back to this module)
