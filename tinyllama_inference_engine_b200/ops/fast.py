"""The bfloat16 serving kernels: tensor-core matrix products and attention.

Kept apart from the core set because they are specialised (by head size, by shape)
and compiled only for what a model needs.
"""
from __future__ import annotations

import functools
import os
import weakref
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..errors import KernelError
from .build import build_library, load_library

library_gemm_calls = 0  # vendor-library matrix products issued (not this engine's kernels)


@functools.lru_cache(maxsize=None)
def sm_count() -> int:
    """Streaming multiprocessors of the current CUDA device (148 on a B200, which is also the answer without a device)."""
    if torch.cuda.is_available():
        return int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
    return 148

DEFAULT_HEAD_DIMS = (64, 128)
_scratch: dict[torch.device, list[torch.Tensor]] = {}


def build_all() -> list:
    built = [build_library(f"tlie_attn_decode_d{d}", ["attention_decode.cu"], {"HEAD_DIM": d}) for d in DEFAULT_HEAD_DIMS]
    built.append(build_library("tlie_attn_decode_d64_w4", ["attention_decode.cu"], {"HEAD_DIM": 64, "DECODE_WARPS": 4, "DECODE_STAGES": 3}))
    built += [build_library(f"tlie_attn_prefill_d{d}", ["attention_prefill.cu"], {"HEAD_DIM": d}) for d in DEFAULT_HEAD_DIMS]
    built.append(build_library("tlie_gemv_fused", ["gemv_fused.cu"]))
    built.append(build_library("tlie_gemm_skinny", ["gemm_skinny.cu"]))
    built.append(build_library("tlie_gemm_tcgen05", TCGEN05_SOURCES))
    built.append(build_library("tlie_attn_prefill_tc", ["attention_prefill_tc.cu"]))
    built.append(build_library("tlie_probes", ["probes.cu"]))
    return built


_ops_module = None


def _ops():
    global _ops_module
    if _ops_module is None:
        from .. import ops

        _ops_module = ops
    return _ops_module


GEMV_KERNEL_MAX_ROWS = 16   # what gemv_fused.cu can take
# Up to this many rows a step uses the fused decode kernels (norm + product, product + residual add, gate).  Measured on the
# 1.1B shapes, a decode step of 9 / 12 / 16 requests: 1.10 / 1.15 / 1.20 ms on them, 1.14 / 1.20 / 1.23 to 1.30 ms on the
# library's product with separate norm and activation kernels.  (With four weight blocks in flight per thread instead of
# eight in the 16-row kernels that read x directly, the fused step took 1.34 to 1.49 ms and lost.)
FUSED_MAX_ROWS = 16
_EPILOGUES = {"store": None, "accumulate": 2, "gated": 3}


def gemv_library():
    return load_library("tlie_gemv_fused", ["gemv_fused.cu"])


def gemv_fits(rows: int, K: int, norm: bool, gated: bool = False, N: int | None = None) -> bool:
    """Whether the fused kernel's shared memory (x as bfloat16 and the warps' partial tiles) fits.

    ``N`` (plain bfloat16 x only): with no more 16-row tiles than the kernel has CTA slots, every CTA computes one tile, uses each
    element of x once and reads it straight from global memory: nothing of x is staged, and any K fits (the down projection of
    wide models: K = 14,336 would need 229 KB for eight staged rows)."""
    if rows > GEMV_KERNEL_MAX_ROWS or K % 8 != 0:
        return False
    if not norm and not gated and N is not None and -(-N // 16) <= 2 * sm_count():
        return True
    padded_rows = 8 if rows <= 8 else 16
    stride = K + ((32 - K % 64) + 64) % 64
    stride += 64 if stride == K else 0
    need = padded_rows * stride * 2 + 8 * 16 * (padded_rows + 1) * 4
    return need <= 200 * 1024


def prepared_norm_buffers(rows: int, width: int, device) -> tuple:
    """Where a product that completes the residual leaves the next norm's input: bfloat16(residual * norm weight) [rows, width]
    and the rows' sums of squares per 16 columns, 32-bit [rows, ceil(width / 16)]."""
    return (torch.empty((rows, width), dtype=torch.bfloat16, device=device), torch.empty((rows, -(-width // 16)), dtype=torch.float32, device=device))


def gemv_fused(x, weight, out, *, norm=None, epilogue: str = "store", prepared=None, prepare=None) -> None:
    """out (+)= f(x) . weight^T for up to 16 rows, one kernel.

    norm      None: ``x`` is bfloat16 [M, K].  (norm_weight, eps, rows): ``x`` is the 32-bit residual stream and
              the operand is rmsnorm(x[rows]) * norm_weight (rows None: the first M rows).
    prepared  (squares, eps): ``x`` is bfloat16(residual * norm weight) [M, K] and ``squares`` [M, tiles] the rows' sums of
              squares, as an earlier "accumulate" with ``prepare`` left them; the operand is the same rmsnorm.
    epilogue  "store": out [M, N] bfloat16 or 32-bit;  "accumulate": out is the 32-bit residual, out += result;
              "gated": weight is [gate rows | up rows], out [M, N / 2] = silu(gate) * up.
    prepare   ("accumulate" only) (norm_weight [N], x_out bfloat16 [M, N], squares_out [M, ceil(N / 16)]): also store
              bfloat16(out * norm_weight) and the rows' sums of squares per 16 columns, for a later call with ``prepared``.
    """
    ops = _ops()
    N, K = weight.shape
    M = out.shape[0]
    if weight.dtype != torch.bfloat16 or M > GEMV_KERNEL_MAX_ROWS or K % 8 != 0:
        raise KernelError(f"gemv_fused takes bfloat16 weights with K % 8 == 0 and at most {GEMV_KERNEL_MAX_ROWS} rows", code="invalid_shape")
    code = _EPILOGUES[epilogue]
    if epilogue == "store":
        code = 1 if out.dtype == torch.float32 else 0
    elif epilogue == "accumulate" and out.dtype != torch.float32:
        raise KernelError("gemv_fused accumulates into the 32-bit residual only", code="invalid_dtype")
    if out.shape[1] != (N // 2 if epilogue == "gated" else N):
        raise KernelError("gemv_fused: the output's width does not fit the weight", code="invalid_shape")
    consume = (c_void_p(0), c_int(0))
    if prepared is not None:
        squares, eps = prepared
        if x.dtype != torch.bfloat16 or x.shape != (M, K) or not x.is_contiguous() or squares.dtype != torch.float32 or squares.shape[0] != M or not squares.is_contiguous():
            raise KernelError("gemv_fused: a prepared norm is bfloat16 [M, K] with 32-bit sums of squares [M, tiles]", code="invalid_shape")
        args = (c_int(3), ops._ptr(x), c_int(K), c_void_p(0), c_void_p(0), c_float(eps))
        consume = (ops._ptr(squares), c_int(squares.shape[1]))
    elif norm is None:
        if x.dtype != torch.bfloat16 or x.shape != (M, K) or x.stride(1) != 1 or x.stride(0) % 8 != 0:
            raise KernelError("gemv_fused: x must be bfloat16 [M, K] with rows 16-byte aligned", code="invalid_shape")
        args = (c_int(0), c_void_p(x.data_ptr()), c_int(x.stride(0)), c_void_p(0), c_void_p(0), c_float(0.0))
    else:
        norm_weight, eps, rows = norm
        if x.dtype != torch.float32 or x.shape[1] != K or norm_weight.dtype != torch.float32 or norm_weight.numel() != K:
            raise KernelError("gemv_fused: the residual and the norm weight must be 32-bit and K wide", code="invalid_shape")
        args = (c_int(1), ops._ptr(x), c_int(K), ops._i32(rows, "rows"), ops._ptr(norm_weight), c_float(eps))
    if not out.is_cuda:
        raise KernelError("this engine has no CPU path: a kernel was given a tensor that is not on a CUDA device")
    emit = (c_void_p(0), c_void_p(0), c_void_p(0))
    if prepare is not None:
        norm_weight, x_out, squares_out = prepare
        if (epilogue != "accumulate" or norm_weight.dtype != torch.float32 or norm_weight.numel() != N or x_out.dtype != torch.bfloat16 or x_out.shape != (M, N)
                or squares_out.dtype != torch.float32 or squares_out.shape != (M, -(-N // 16)) or not x_out.is_contiguous() or not squares_out.is_contiguous()):
            raise KernelError("gemv_fused: prepare takes a 32-bit norm weight [N], bfloat16 [M, N] and 32-bit [M, ceil(N / 16)], with accumulate", code="invalid_shape")
        emit = (ops._ptr(norm_weight), ops._ptr(x_out), ops._ptr(squares_out))
    ops._check(gemv_library().tlie_gemv_fused(*args, ops._ptr(weight), ops._ptr(out), c_int(M), c_int(N), c_int(K), c_int(code), *consume, *emit, ops._stream()),
               "gemv_fused")


# --- tensor-core product for 17 to 127 rows (tcgen05 with the operands swapped, K cut over a cluster) -----------------
SKINNY_MAX_ROWS = 127      # steps of more rows than the register-fed kernels take and fewer than a 128-row tile
# Off unless asked for (``enable_skinny`` or TLIE_SKINNY=1).  Measured on the 1.1B shapes, a decode step of 24 / 32 / 64 requests:
# 1.28 / 1.28 / 1.64 ms with this kernel and its fusions against 1.14 / 1.15 / 1.29 ms on the library's products with separate
# norm and activation kernels.  Its tiles are few (10 for 2,560 weight rows), so K is cut over a cluster, and what the CTAs then
# exchange (64 rows x 256 columns of 32-bit partial sums each) is half as many bytes as the weights they read.
use_skinny = False


def enable_skinny(on: bool = True) -> None:
    """Route products of 17 to 127 rows (and what surrounds them: norm in front, gate or residual add behind) to ``gemm_skinny``."""
    global use_skinny, FUSED_MAX_ROWS
    use_skinny = bool(on)
    FUSED_MAX_ROWS = SKINNY_MAX_ROWS if on else GEMV_KERNEL_MAX_ROWS


_SKINNY_EPILOGUES = {"store": None, "gated": 2, "accumulate": 3}


def skinny_library():
    return load_library("tlie_gemm_skinny", ["gemm_skinny.cu"])


def skinny_fits(rows: int, weight, x=None) -> bool:
    """Whether ``gemm_skinny`` takes a product of this many rows with this weight (and this x, if given)."""
    if not 1 <= rows <= SKINNY_MAX_ROWS or weight.dtype != torch.bfloat16 or weight.shape[1] % 8 != 0 or not weight.is_contiguous():
        return False
    return x is None or (x.dtype == torch.bfloat16 and x.is_contiguous() and x.data_ptr() % 16 == 0)


_skinny_packed: dict[tuple, tuple] = {}


def skinny_packed(weight: torch.Tensor, gated: bool = False) -> torch.Tensor:
    """The copy of ``weight`` that ``gemm_skinny`` streams: its 128 x 64 operand tiles, each as the contiguous 16 KB image the tensor
    cores read from shared memory (``gated``: a group is 64 gate rows and the 64 up rows of the same outputs).  Made on first use and
    kept for as long as the weight tensor lives: weights do not change, and a captured graph keeps pointing at the copy.  The entry
    is tied to the tensor object itself (an address alone could be handed to another tensor once this one is freed)."""
    key = (weight.data_ptr(), tuple(weight.shape), bool(gated), weight.device)
    found = _skinny_packed.get(key)
    if found is not None and found[0]() is weight:
        return found[1]
    ops = _ops()
    N, K = weight.shape
    library = skinny_library()
    if not getattr(library, "_tlie_typed", False):
        library.tlie_gemm_skinny_packed_elements.restype = c_longlong
        library._tlie_typed = True
    elements = library.tlie_gemm_skinny_packed_elements(c_int(N), c_int(K), c_int(1 if gated else 0))
    packed = torch.empty(elements, dtype=torch.bfloat16, device=weight.device)
    ops._check(library.tlie_gemm_skinny_pack(ops._ptr(weight), ops._ptr(packed), c_int(N), c_int(K), c_int(1 if gated else 0), ops._stream()), "gemm_skinny_pack")
    _skinny_packed[key] = (weakref.ref(weight, lambda _, key=key: _skinny_packed.pop(key, None)), packed)
    return packed


def skinny_square_runs(rows: int, N: int, K: int) -> int:
    """Partial sums of squares per row that ``gemm_skinny(..., prepare=)`` leaves for a [N, K] weight and this many rows."""
    return int(skinny_library().tlie_gemm_skinny_square_runs(c_int(rows), c_int(N), c_int(K)))


def gemm_skinny(x, weight, out, *, epilogue: str = "store", prepared=None, prepare=None) -> None:
    """out (+)= x . weight^T for up to 128 rows on the tensor cores, the weights streamed once; one kernel.

    x         bfloat16 [M, K], contiguous.
    prepared  (squares, eps): x is bfloat16(residual * norm weight) and ``squares`` [M, runs] (rows may be strided) partial sums of
              squares of the residual's rows; every result is scaled by its row's 1 / sqrt(mean + eps) (not with "accumulate").
    epilogue  "store": out [M, N] bfloat16 or 32-bit; "gated": weight is [gate rows | up rows], out [M, N / 2] = silu(gate) * up;
              "accumulate": out is the 32-bit residual [M, N], out += result.
    prepare   ("accumulate" only) (norm_weight [N], x_out bfloat16 [M, N], squares_out [M, skinny_square_runs(M, N, K)], rows may be
              strided): also leave the next norm's input, for a later call with ``prepared``.
    """
    ops = _ops()
    N, K = weight.shape
    M = x.shape[0]
    if not skinny_fits(M, weight, x) or x.shape[1] != K:
        raise KernelError(f"gemm_skinny takes contiguous bfloat16 operands with K % 8 == 0 and at most {SKINNY_MAX_ROWS + 1} rows", code="invalid_shape")
    code = _SKINNY_EPILOGUES[epilogue]
    if epilogue == "store":
        if out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError("gemm_skinny stores bfloat16 or 32-bit", code="invalid_dtype")
        code = 1 if out.dtype == torch.float32 else 0
    elif epilogue == "accumulate" and out.dtype != torch.float32:
        raise KernelError("gemm_skinny accumulates into the 32-bit residual only", code="invalid_dtype")
    elif epilogue == "gated" and (out.dtype != torch.bfloat16 or N % 2):
        raise KernelError("gemm_skinny: a gated product stores bfloat16 and its weight has an even number of rows", code="invalid_shape")
    if out.shape != (M, N // 2 if epilogue == "gated" else N) or not out.is_contiguous():
        raise KernelError("gemm_skinny: the output's shape does not fit the weight", code="invalid_shape")
    consume = (c_void_p(0), c_int(0), c_int(0), c_float(0.0))
    if prepared is not None:
        squares, eps = prepared
        if epilogue == "accumulate" or squares.dtype != torch.float32 or squares.dim() != 2 or squares.shape[0] != M or squares.stride(1) != 1 or not squares.is_cuda:
            raise KernelError("gemm_skinny: a prepared norm brings 32-bit sums of squares [M, runs], and not with accumulate", code="invalid_shape")
        consume = (c_void_p(squares.data_ptr()), c_int(squares.shape[1]), c_int(squares.stride(0)), c_float(eps))
    emit = (c_void_p(0), c_void_p(0), c_void_p(0), c_int(0))
    if prepare is not None:
        norm_weight, x_out, squares_out = prepare
        if (epilogue != "accumulate" or norm_weight.dtype != torch.float32 or norm_weight.numel() != N or x_out.dtype != torch.bfloat16 or x_out.shape != (M, N)
                or squares_out.dtype != torch.float32 or squares_out.dim() != 2 or squares_out.shape != (M, skinny_square_runs(M, N, K)) or squares_out.stride(1) != 1
                or not x_out.is_contiguous() or not squares_out.is_cuda):
            raise KernelError("gemm_skinny: prepare takes a 32-bit norm weight [N], bfloat16 [M, N] and 32-bit [M, skinny_square_runs(M, N, K)], with accumulate", code="invalid_shape")
        emit = (ops._ptr(norm_weight), ops._ptr(x_out), c_void_p(squares_out.data_ptr()), c_int(squares_out.stride(0)))
    ops._check(skinny_library().tlie_gemm_skinny(ops._ptr(x), ops._ptr(skinny_packed(weight, epilogue == "gated")), ops._ptr(out), c_int(M), c_int(N), c_int(K), c_int(code),
                                                 *consume, *emit, ops._ptr(tcgen05_error_flag(x.device)), ops._stream()), "gemm_skinny")


# --- tensor-core product for many rows (tcgen05, TMA, tensor memory) -------------------------------------
# Where the engine's own tcgen05 kernels run instead of the library's product (and, for the fused forms, the small kernel after
# it).  Measured with CUDA events in a replayed graph, weights from HBM, at 1.1B, 7B and 8B widths, 128 to 8,192 rows
# (`kernel-bench --products`): the engine's kernels are level with or ahead of the library wherever their tiles are wide and keep the
# SMs busy over whole waves and the product is large enough for its start and end not to count, and behind elsewhere, since a CTA
# runs all of K for its tile where the library also splits K:
#   * 1.1B widths, 2,048 rows: qkv 19.9 us (one wave of 288-wide tiles) against 19.0, o (adding) 17.5 against 22.0 for product + add
#     kernel; 1,024 rows: qkv 14.7 against 10.9 (half the work, the same start and end), o 16.5 against 14.1 (32 tiles for 74 pairs);
#   * 7B widths, 1,024 rows: o 28.1 against 33.8, down 67.3 against 71.2, qkv level; 8B widths, 1,024 rows: qkv 44.8 against 37.4 (96
#     tiles for 74 pairs: two waves, the second a third full);
#   * the gated product on pairs of SMs is ahead of product + activation kernel from 1,024 rows on (7B widths: 130 against
#     160 us; 1.1B widths: 46.7 against 45.5); below that it is ahead where the product is a large one (7B widths, 768 rows: 104
#     against 112 us; 8B widths, 512 rows: 100 against 112) and behind where it is not (1.1B widths, 768 rows: 36.4 against 34.5).
TCGEN05_MIN_ROWS = 1024            # below this the library was ahead at every width
TCGEN05_GATED_MIN_ROWS = 1024
TCGEN05_GATED_LARGE = (512, 80e9)  # the gated product also from this many rows on where it is this many flop or more
OWN_PRODUCT_MIN_EFFICIENCY = 0.75  # what the product's tiling costs against 256-wide tiles on every SM with no wave left partly empty (0.76: ahead, 0.73: behind)
OWN_PRODUCT_MIN_FLOP = 20e9        # a smaller product is mostly its start and end, where the library is ahead
OWN_ADDING_MIN_FLOP = 10e9         # the adding product also saves the add kernel
use_tcgen05 = True


TCGEN05_SOURCES = ["gemm_tcgen05.cu", "gemm_tcgen05_pair.cu"]


def tcgen05_takes(M: int, N: int, K: int, adding: bool = False) -> bool:
    """Whether a plain product (``adding``: one that adds into the residual) runs on this engine's tcgen05 kernels (else on the
    library's): from TCGEN05_MIN_ROWS rows on, where the tiling it would get is an efficient one (waves that are full, tiles that
    are not narrow: the cost model of ``_cheapest_tiles`` against its own ideal) and the product is not a small one.

    (Sharing a tile's k blocks among CTAs, which would fill the SMs for small products too, was tried in the one-SM kernel: the
    owner of a tile collects the others' partial accumulators at the very end of its share, eight trips to the L2 per partial
    tile with nothing left to hide them behind, and that cost more than even shares saved.)"""
    if M < TCGEN05_MIN_ROWS:
        return False
    pair = (use_sm_pairs and M >= PAIR_MIN_ROWS) if adding else pair_tiles_pay(M, N)
    _, cost, _ = _cheapest_tiles(M, N, pair, adding)
    ideal = -(-M // (256 if pair else 128)) * N / (sm_count() // 2 if pair else sm_count()) * (256 + 300) / 256
    return ideal / cost >= OWN_PRODUCT_MIN_EFFICIENCY and 2.0 * M * N * K >= (OWN_ADDING_MIN_FLOP if adding else OWN_PRODUCT_MIN_FLOP)


def gated_takes(M: int, N: int, K: int) -> bool:
    """Whether the gated product ([gate rows | up rows]: N rows of w in all) of a step of M rows runs on this engine's tcgen05 kernel."""
    return M >= TCGEN05_GATED_MIN_ROWS or (M >= TCGEN05_GATED_LARGE[0] and 2.0 * M * N * K >= TCGEN05_GATED_LARGE[1])


def tcgen05_library():
    return load_library("tlie_gemm_tcgen05", TCGEN05_SOURCES)


def tcgen05_error_flag(device: torch.device) -> torch.Tensor:
    """The device's error word: the tensor-core kernels set bit 0 of it if one of their bounded waits gave up."""
    return _ops().error_flag(device)


GEMM_TILE_WIDTHS = (256, 192, 160, 128)
GEMM_WIDE_TILES = (288, 320)   # two MMAs wide, one accumulator: for products that fit one wave of CTAs so (one-SM tiles only)


# Tiles of 256 rows on pairs of SMs (tcgen05 cta_group::2, gemm_tcgen05_pair.cu) bring a third less from L2 per flop.  That pays
# where a product is several waves of tiles, so that what the SMs can pull from L2 sets the pace: measured at 2,048 rows and
# K = 4,096, N = 12,288: 139 us on pairs, 153 on single SMs (the library: 142); N = 4,096, K = 11,008: 129, 163 (144); 8,192 rows,
# N = 6,144: 278, 317 (278).  The pairs have wide tiles of their own (two MMAs wide, one accumulator) for products that fit one
# wave of the pairs so: 2,048 x 4,096 is 128 tiles of 256 columns for 74 pairs, or 72 tiles of 480 (K = 11,008, adding into the
# residual: 132 -> 123.5 us; 2,048 x 3,072 x 3,072 with 384-wide tiles: 42.7 -> 36.6 us).  The gated product runs on pairs from
# 1,024 rows.
PAIR_MIN_ROWS = 1024
PAIR_TILE_WIDTHS = (256,)          # narrower tiles on pairs were behind the 256-wide ones wherever they were measured
PAIR_WIDE_TILES = (288, 384, 480)
PAIR_ADDING_WIDE_TILES = (384, 480)
PAIR_TILE_GAIN = 0.9               # a tile on a pair of SMs against two tiles of the same width on single SMs, where L2 sets the pace
use_sm_pairs = True


def _cheapest_tiles(M: int, N: int, pair: bool, adding: bool) -> tuple[int, int, int]:
    """(tile width, cost, waves) of the cheapest way to tile an M x N product on single SMs or on pairs: cost = waves x (width + 300).

    A tile costs its width plus a fixed part about as large as 300 columns (measured: a 128 x 160 tile takes 0.8 of the time
    of a 128 x 256 one), so the widest tile wins unless a narrower one saves a whole wave; the wider tile on a tie.  A wide
    tile has no second accumulator to work on while its epilogue runs, so it is a candidate only where no CTA gets two."""
    workers = sm_count() // 2 if pair else sm_count()
    row_blocks = -(-M // (256 if pair else 128))
    if pair:
        widths, wide = PAIR_TILE_WIDTHS, (PAIR_ADDING_WIDE_TILES if adding else PAIR_WIDE_TILES)
    else:
        widths, wide = ((256,), ()) if adding else (GEMM_TILE_WIDTHS, GEMM_WIDE_TILES)
    candidates = tuple(width for width in wide if row_blocks * -(-N // width) <= workers) + widths
    waves = lambda width: -(-(row_blocks * -(-N // width)) // workers)  # noqa: E731
    best = min(candidates, key=lambda width: (waves(width) * (width + 300), -width))
    return best, waves(best) * (best + 300), waves(best)


@functools.lru_cache(maxsize=4096)
def gemm_tile_width(M: int, N: int, pair: bool = False, adding: bool = False) -> int:
    """The tile width whose waves of persistent CTAs (or pairs of them) cost least; ``adding``: for the product that adds into the residual."""
    return _cheapest_tiles(M, N, pair, adding)[0]


@functools.lru_cache(maxsize=4096)
def pair_tiles_pay(M: int, N: int) -> bool:
    """Whether a plain product of this shape runs on pairs of SMs: where their cheapest tiling (with what a pair gains on two single
    SMs, if it is waves of tiles) costs less than the cheapest one-SM tiling; a product that one wave of one-SM tiles holds stays there."""
    if not use_sm_pairs or M < PAIR_MIN_ROWS:
        return False
    _, pair_cost, pair_waves = _cheapest_tiles(M, N, True, False)
    return (PAIR_TILE_GAIN if pair_waves > 1 else 1.0) * pair_cost < _cheapest_tiles(M, N, False, False)[1]


def gemm_tcgen05(x, weight, out, tile_n: int | None = None, pair: bool | None = None) -> None:
    """out[M, N] = x[M, K] . weight[N, K]^T on the 5th-generation tensor cores; bfloat16 in, bfloat16 or 32-bit out.

    ``pair``: 256-row tiles on pairs of SMs (each CTA loads half of the weight rows of a tile)."""
    ops = _ops()
    M, K = x.shape
    N = weight.shape[0]
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or K % 8 != 0 or not x.is_contiguous():
        raise KernelError("gemm_tcgen05 takes contiguous bfloat16 operands with K % 8 == 0", code="invalid_shape")
    if pair is None:
        pair = tile_n is None and pair_tiles_pay(M, N)
    if tile_n is None:
        tile_n = gemm_tile_width(M, N, pair)
    library = tcgen05_library()
    entry = library.tlie_gemm_tcgen05_pair if pair else library.tlie_gemm_tcgen05
    ops._check(
        entry(ops._ptr(x), ops._ptr(weight), ops._ptr(out), c_int(M), c_int(N), c_int(K), c_int(1 if out.dtype == torch.float32 else 0),
              c_int(tile_n), ops._ptr(tcgen05_error_flag(x.device)), ops._stream()),
        "gemm_tcgen05",
    )


use_accumulate_epilogue = True   # o-proj and down-proj of prompt portions add into the residual from the product's epilogue


def can_accumulate(rows: int, weight) -> bool:
    """Whether ``gemm_tcgen05_accumulate`` takes residual += x . weight^T for this many rows."""
    N, K = weight.shape
    return (use_tcgen05 and use_accumulate_epilogue and weight.dtype == torch.bfloat16 and N % 4 == 0 and K % 8 == 0 and tcgen05_takes(rows, N, K, adding=True))


def gemm_tcgen05_accumulate(x, weight, residual, pair: bool | None = None, tile_n: int | None = None) -> None:
    """residual[M, N] (32-bit) += x[M, K] . weight[N, K]^T: the product's tiles are added by bulk tensor reductions, each element once.

    ``pair``: on pairs of SMs (default: from PAIR_MIN_ROWS rows on; these tiles are 256 wide either way, and the pairs were ahead
    at every shape measured: down-proj of 2,048 rows at 1.1B widths 38.4 -> 35.3 us, at 7B widths 146 -> 133, at 8B widths and
    8,192 rows 749 -> 668)."""
    ops = _ops()
    M, K = x.shape
    N = weight.shape[0]
    if (x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or residual.dtype != torch.float32 or residual.shape != (M, N) or K % 8 != 0 or N % 4 != 0
            or not x.is_contiguous() or not residual.is_contiguous()):
        raise KernelError("gemm_tcgen05_accumulate takes contiguous bfloat16 operands (K % 8 == 0) and a contiguous 32-bit residual [M, N] with N % 4 == 0", code="invalid_shape")
    if pair is None:
        pair = use_sm_pairs and M >= PAIR_MIN_ROWS
    if tile_n is None:
        tile_n = gemm_tile_width(M, N, pair, adding=True)
    library = tcgen05_library()
    entry = library.tlie_gemm_tcgen05_pair if pair else library.tlie_gemm_tcgen05
    ops._check(
        entry(ops._ptr(x), ops._ptr(weight), ops._ptr(residual), c_int(M), c_int(N), c_int(K), c_int(3), c_int(tile_n),
              ops._ptr(tcgen05_error_flag(x.device)), ops._stream()),
        "gemm_tcgen05_accumulate",
    )


def gemm_tcgen05_gated(x, weight, out, pair: bool | None = None) -> None:
    """out[M, I] = silu(x . gate^T) * (x . up^T) for weight = [gate rows | up rows] ([2 I, K]), one kernel."""
    ops = _ops()
    M, K = x.shape
    inter = weight.shape[0] // 2
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or K % 8 != 0 or not x.is_contiguous() or out.shape != (M, inter):
        raise KernelError("gemm_tcgen05_gated takes contiguous bfloat16 operands with K % 8 == 0 and out [M, rows / 2]", code="invalid_shape")
    if pair is None:   # below the pairs' usual row count: where the rows are whole 256-row tiles (640 rows at 7B widths: 102 us on pairs, 96 on single SMs)
        pair = use_sm_pairs and (M >= PAIR_MIN_ROWS or (M >= 512 and M % 256 == 0))
    library = tcgen05_library()
    entry = library.tlie_gemm_tcgen05_pair if pair else library.tlie_gemm_tcgen05
    ops._check(
        entry(ops._ptr(x), ops._ptr(weight), ops._ptr(out), c_int(M), c_int(inter), c_int(K), c_int(2), c_int(256),
              ops._ptr(tcgen05_error_flag(x.device)), ops._stream()),
        "gemm_tcgen05_gated",
    )


def linear_bf16(x, weight, out) -> None:
    global library_gemm_calls
    if weight.dtype != torch.bfloat16 or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("linear: the bfloat16 path takes bfloat16 weights", code="invalid_dtype")
    if x.stride(0) % 8 == 0 and gemv_fits(x.shape[0], weight.shape[1], norm=False, N=weight.shape[0]):
        gemv_fused(x, weight, out)
        return
    if use_tcgen05 and tcgen05_takes(x.shape[0], weight.shape[0], weight.shape[1]) and weight.shape[1] % 8 == 0 and x.is_contiguous():
        gemm_tcgen05(x, weight, out)
        return
    if use_skinny and skinny_fits(x.shape[0], weight, x) and out.is_contiguous():
        gemm_skinny(x, weight, out)
        return
    library_gemm_calls += 1
    if out.dtype == torch.float32:
        torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
    else:
        torch.mm(x, weight.t(), out=out)


# --- decode attention -------------------------------------------------------------------------
def decode_attention_library(head_dim: int, narrow: bool = False):
    """The decode attention library of a head size.

    Default build: eight warps and two stages per CTA for head sizes up to 64 (one CTA per SM pulls enough bandwidth when
    there are few (request, kv head) pairs).  ``narrow``: four warps and three stages, two CTAs per SM, for steps with
    more pairs than SMs, where the wide CTAs would run in two uneven waves.
    """
    if narrow and head_dim <= 64:
        lib = load_library(f"tlie_attn_decode_d{head_dim}_w4", ["attention_decode.cu"], {"HEAD_DIM": head_dim, "DECODE_WARPS": 4, "DECODE_STAGES": 3})
    else:
        lib = load_library(f"tlie_attn_decode_d{head_dim}", ["attention_decode.cu"], {"HEAD_DIM": head_dim})
    if not getattr(lib, "_tlie_typed", False):
        lib.tlie_decode_attention_scratch_floats.restype = c_longlong
        lib._tlie_typed = True
    return lib


def decode_splits(requests: int, kv_heads: int, max_context: int) -> int:
    """Parts the key range is cut into: at most one CTA (eight warps) per SM, at least 256 keys per part, at most 32 parts."""
    by_occupancy = max(1, sm_count() // max(1, requests * kv_heads))   # rounded down: one CTA too many is a second wave
    by_length = max(1, -(-max_context // 256))
    return max(1, min(by_occupancy, by_length, 32))


def scratch(device: torch.device, floats: int) -> torch.Tensor:
    """Scratch memory of stable address (captured graphs keep pointing at it): grown, never freed."""
    held = _scratch.setdefault(device, [])
    if not held or held[-1].numel() < floats:
        held.append(torch.zeros(max(floats, 1 << 20), dtype=torch.float32, device=device))  # zero: it starts with the merge counters
    return held[-1]


def decode_attention(qkv, pages, positions, block_table, out, q_heads: int, kv_heads: int, head_dim: int, page_size: int,
                     window: int, scale: float, splits: int, fuse_rope: bool = False, inv_freq=None, write_cache: bool = True) -> None:
    """One query token per request (row i of qkv belongs to request i) over its cached keys; bfloat16.

    ``fuse_rope``: the rows of qkv are the unrotated [q | k | v] of the new tokens; the kernel rotates q and k with
    ``inv_freq`` (None: no rotation) and, with ``write_cache``, stores the new key and value in the request's page.
    """
    ops = _ops()
    requests = qkv.shape[0]
    lib = decode_attention_library(head_dim, narrow=requests * kv_heads > sm_count())
    floats = lib.tlie_decode_attention_scratch_floats(c_int(requests), c_int(q_heads), c_int(splits))
    buffer = scratch(qkv.device, floats)
    ops._check(
        lib.tlie_decode_attention(
            ops._ptr(qkv), c_int(qkv.shape[1]), ops._ptr(pages), ops._i32(positions, "positions"), ops._i32(block_table, "block_table"),
            c_int(block_table.shape[1]), ops._ptr(out), ops._ptr(buffer), c_int(requests), c_int(q_heads), c_int(kv_heads), c_int(page_size),
            c_int(window), c_float(scale), c_int(splits), c_int(1 if fuse_rope else 0), ops._ptr(inv_freq), c_int(1 if write_cache else 0), ops._stream(),
        ),
        "decode_attention",
    )


def can_fuse_rope_into_decode(batch, qkv, head_dim: int, q_heads: int, kv_heads: int, inv_freq, rotary_dim: int) -> bool:
    """Whether a decode step's rotation and cache write can happen inside the attention kernel."""
    if batch is None or qkv.dtype != torch.bfloat16 or not batch.decode_only or qkv.shape[0] != batch.num_seqs:
        return False
    if head_dim % 16 != 0 or head_dim > 128 or q_heads // kv_heads > 16 or batch.num_seqs * kv_heads > 16384:
        return False
    return inv_freq is None or (rotary_dim == head_dim and head_dim % 32 == 0)


# --- prompt (and mixed) attention -----------------------------------------------------------------
ATTENTION_TILE_ROWS = 64       # rows of one work item of the mma.sync prompt kernel (csrc/attention_prefill.cu: PREFILL_ROWS)
ATTENTION_TC_TILE_ROWS = 128   # rows of one work item of the tensor-memory kernel (csrc/attention_prefill_tc.cu)


def leading_single_rows(q_lens: list[int]) -> int:
    """How many entries at the head of a step bring one token each (the scheduler puts the decoding requests first).  In a step
    that also carries prompt portions these rows go to the decode kernel (split keys, a CTA per part) and the work lists of the
    prompt kernels leave them out: as 1-row tiles of a prompt kernel each of them cost a whole tile's pass over its keys, and
    enough of them took the step off the tensor-memory kernel altogether."""
    lead = 0
    while lead < len(q_lens) and q_lens[lead] == 1:
        lead += 1
    return lead if lead < len(q_lens) else 0


def attention_tiles(q_lens: list[int], first_positions: list[int], seq_starts: list[int], first_entry: int = 0, end_entry: int | None = None) -> list[int]:
    """Work items of the mma.sync prompt kernel: (entry, first row) of every run of up to ATTENTION_TILE_ROWS rows of one entry."""
    tiles: list[int] = []
    for index in range(first_entry, len(q_lens) if end_entry is None else end_entry):
        for offset in range(0, q_lens[index], ATTENTION_TILE_ROWS):
            tiles += [index, seq_starts[index] + offset]
    return tiles


def _row_tiles_by_work(q_lens: list[int], first_positions: list[int], seq_starts: list[int], first_entry: int) -> list[tuple[int, int, int]]:
    """(key tiles it sees, entry, first row) of every run of ATTENTION_TC_TILE_ROWS rows, the heaviest first."""
    singles = []
    for index in range(first_entry, len(q_lens)):
        count = q_lens[index]
        for offset in range(0, count, ATTENTION_TC_TILE_ROWS):
            rows = min(ATTENTION_TC_TILE_ROWS, count - offset)
            work = -(-(first_positions[index] + offset + rows) // 64)
            singles.append((work, index, seq_starts[index] + offset))
    singles.sort(key=lambda item: -item[0])
    return singles


def paired_attention_tiles(q_lens: list[int], first_positions: list[int], seq_starts: list[int], first_entry: int = 0) -> list[int]:
    """Work items of two row tiles for the tensor-memory attention kernel: (entry, first row, entry or -1, first row) per item.

    A run of ATTENTION_TC_TILE_ROWS rows late in a long request sees many keys, an early one few.  Pairing the heaviest
    tile with the lightest, the second heaviest with the second lightest, and so on, gives every CTA about the same
    number of key tiles.  The kernel takes such items, but steps do not send them: a CTA is a chain of dependent waits,
    so twice the CTAs with half the work each are faster at every length (one request of 512 tokens at 32 heads of 64:
    15.6 us in pairs, 11.9 us as single tiles; 1,024: 25.7 / 21.1; 2,048: 42.5 / 41.2; 4,096: 139 / 129; head size 128, 2,048:
    60.9 / 54.1).  Kept for the kernel's tests and its cycle counters."""
    singles = _row_tiles_by_work(q_lens, first_positions, seq_starts, first_entry)
    flat: list[int] = []
    low, high = 0, len(singles) - 1
    while low <= high:
        _, index, row = singles[low]
        if low < high:
            _, index2, row2 = singles[high]
            flat += [index, row, index2, row2]
        else:
            flat += [index, row, -1, 0]
        low += 1
        high -= 1
    return flat


def single_attention_tiles(q_lens: list[int], first_positions: list[int], seq_starts: list[int], first_entry: int = 0) -> list[int]:
    """Work items of the tensor-memory attention kernel, a row tile each, heaviest first: (entry, first row, -1, 0) per item.  The CTAs
    are handed out in this order, so every slot that comes free takes the heaviest tile left."""
    flat: list[int] = []
    for _, index, row in _row_tiles_by_work(q_lens, first_positions, seq_starts, first_entry):
        flat += [index, row, -1, 0]
    return flat


def _register_step_plans() -> None:
    """The prompt-attention kernels' work lists travel with every step that is not pure decoding (engine.batch.register_step_plan).

    They leave out the decoding requests at the head of the step (``leading_single_rows``); ``attention_tiles_lead`` holds those as
    1-row tiles, for shapes the decode kernel does not take."""
    from ..engine.batch import StepPlan, register_step_plan

    not_decode = lambda q_lens: max(q_lens) > 1  # noqa: E731
    register_step_plan(StepPlan("attention_tiles", 2, lambda q, f, s: attention_tiles(q, f, s, leading_single_rows(q)), not_decode), replace=True)
    register_step_plan(StepPlan("attention_tiles_tc", 4, lambda q, f, s: single_attention_tiles(q, f, s, leading_single_rows(q)), not_decode), replace=True)
    register_step_plan(StepPlan("attention_tiles_lead", 2, lambda q, f, s: attention_tiles(q, f, s, 0, leading_single_rows(q)),
                                lambda q_lens: max(q_lens) > 1 and leading_single_rows(q_lens) > 0), replace=True)


_register_step_plans()


def prefill_attention(qkv, pages, tiles, seq_starts, first_positions, block_table, out, q_heads: int, kv_heads: int, head_dim: int,
                      page_size: int, window: int, scale: float) -> None:
    """Flash attention of every tile in ``tiles`` (int32 [n, 2]: request, first row; up to 128 rows each) over the paged cache; bfloat16."""
    ops = _ops()
    lib = load_library(f"tlie_attn_prefill_d{head_dim}", ["attention_prefill.cu"], {"HEAD_DIM": head_dim})
    ops._check(
        lib.tlie_prefill_attention(
            ops._ptr(qkv), c_int(qkv.shape[1]), ops._ptr(pages), ops._i32(tiles, "tiles"), c_int(tiles.shape[0]), ops._i32(seq_starts, "seq_starts"),
            ops._i32(first_positions, "first_positions"), ops._i32(block_table, "block_table"), c_int(block_table.shape[1]), ops._ptr(out),
            c_int(q_heads), c_int(kv_heads), c_int(page_size), c_int(window), c_float(scale), ops._stream(),
        ),
        "prefill_attention",
    )


use_tc_attention = True    # the tcgen05 / tensor-memory prompt attention (head size 64 or 128, pages of a multiple of 64 keys)
TC_ATTENTION_HEAD_DIMS = (64, 128)
TC_ATTENTION_MIN_ROWS_PER_TILE = 32


def prefill_attention_tc(qkv, pages, tiles, seq_starts, first_positions, block_table, out, q_heads: int, kv_heads: int, head_dim: int, page_size: int,
                         window: int, scale: float) -> None:
    """Flash attention of the work items in ``tiles`` (int32 [n, 4], see ``paired_attention_tiles``) on the 5th-generation tensor cores; head size 64 or 128, bfloat16."""
    ops = _ops()
    if head_dim not in TC_ATTENTION_HEAD_DIMS or page_size % 64 != 0:
        raise KernelError("the tensor-memory attention takes head sizes 64 and 128 and pages of a multiple of 64 keys", code="invalid_shape")
    lib = load_library("tlie_attn_prefill_tc", ["attention_prefill_tc.cu"])
    ops._check(
        lib.tlie_prefill_attention_tc(
            ops._ptr(qkv), c_int(qkv.shape[1]), c_int(qkv.shape[0]), ops._ptr(pages), c_int(pages.shape[0]), ops._i32(tiles, "tiles"), c_int(tiles.shape[0]),
            ops._i32(seq_starts, "seq_starts"), ops._i32(first_positions, "first_positions"), ops._i32(block_table, "block_table"),
            c_int(block_table.shape[1]), ops._ptr(out), c_int(q_heads), c_int(kv_heads), c_int(head_dim), c_int(page_size), c_int(window), c_float(scale),
            ops._ptr(tcgen05_error_flag(qkv.device)), ops._stream(),
        ),
        "prefill_attention_tc",
    )


def paged_attention_bf16(qkv, pages, positions, token_seq, block_table, out, q_heads, kv_heads, head_dim, page_size, window, scale, batch) -> bool:
    """Run a specialised kernel if one covers this shape; False sends the caller to the general one."""
    if batch is None or pages.dtype != torch.bfloat16:
        return False
    if batch.decode_only and qkv.shape[0] == batch.num_seqs and head_dim <= 128 and q_heads // kv_heads <= 16:
        splits = decode_splits(batch.num_seqs, kv_heads, batch.max_seq_len)
        decode_attention(qkv, pages, positions, block_table, out, q_heads, kv_heads, head_dim, page_size, window, scale, splits)
        return True
    if head_dim > 128:
        return False
    lead = leading_single_rows(batch.host_q_lens)
    if lead:   # decoding requests at the head of a step that also carries prompt portions: rows 0 .. lead - 1, one per entry
        if q_heads // kv_heads <= 16:
            decode_attention(qkv[:lead], pages, positions[:lead], block_table[:lead], out[:lead], q_heads, kv_heads, head_dim, page_size, window, scale,
                             decode_splits(lead, kv_heads, batch.max_seq_len))
        else:
            prefill_attention(qkv, pages, batch.plan("attention_tiles_lead"), batch.seq_starts, batch.first_positions, block_table, out, q_heads, kv_heads,
                              head_dim, page_size, window, scale)
    tc_tiles = batch.plan("attention_tiles_tc")
    if (use_tc_attention and tc_tiles is not None and head_dim in TC_ATTENTION_HEAD_DIMS and page_size % 64 == 0 and pages.is_contiguous()
            and batch.num_tokens - lead >= TC_ATTENTION_MIN_ROWS_PER_TILE * tc_tiles.shape[0]):
        prefill_attention_tc(qkv, pages, tc_tiles, batch.seq_starts, batch.first_positions, block_table, out, q_heads, kv_heads, head_dim, page_size, window, scale)
        return True
    tiles = batch.plan("attention_tiles")
    if tiles is not None:
        prefill_attention(qkv, pages, tiles, batch.seq_starts, batch.first_positions, block_table, out, q_heads, kv_heads,
                          head_dim, page_size, window, scale)
        return True
    return False


if os.environ.get("TLIE_SKINNY", "0") == "1":
    enable_skinny(True)
