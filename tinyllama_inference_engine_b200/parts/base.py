"""Interfaces of the parts a model is put together from.

Five categories: ``mixer`` (token mixing: attention here), ``feed_forward``,
``norm``, ``position`` (position encoding) and ``block`` (their arrangement in one
layer); plus ``embedding`` and ``head`` at the ends of the model.  A part is built
from a ``PartSpec`` (its sizes and constants), a tensor-name prefix, the weight
store and the runtime.  No part knows which model it is in.

What each category must offer:

  every part   ``tensor_specs(spec, prefix)`` (classmethod): the tensors it reads.
  norm         ``forward(residual, delta=None, rows=None) -> normed``: adds ``delta``
               into the 32-bit ``residual`` first if given, normalises all rows or
               the rows listed in ``rows``.
  position     ``rotary_table()`` -> (inv_freq, rotary_dim) if the encoding is a
               rotation the fused cache-write kernel can apply, else None, in which
               case ``apply(qkv, ctx, q_heads, kv_heads, head_dim)`` edits q and k in place.
  mixer        ``cache_need(spec)`` (classmethod) -> CacheNeed: pages of keys and
               values, per-request state of fixed size, or nothing;
               ``forward(x, ctx, cache) -> y`` for the step's tokens ``x [T, hidden]``.
  feed_forward ``forward(x, ctx) -> y``.
               (A mixer or feed-forward may set ``accepts_lazy_norm`` / ``fuses_residual_add``
               to take the norm before it and the residual add after it into its own kernels, and
               ``prepares_next_norm`` to take ``prepare=<the lazy norm that follows>`` along with
               ``accumulate_into`` and leave that norm's input for the next product.)
  block        ``forward(residual, pending, ctx, cache) -> (residual, pending)``: the hidden state
               is the pair (32-bit residual, what is pending on it): None, the last output not
               yet added, or (residual complete) a lazy norm already prepared for whoever
               normalises next.  A block with ``accepts_next_norm`` is also given
               ``next_norm=<the norm part that will read its result>``.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..errors import BatchError, ConfigError
from .spec import PartSpec, TensorSpec


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer keeps per request between steps.

    kind "pages": for every cached token (or only the last ``window`` tokens if window > 0) a number of *planes*, each
    ``heads`` vectors of ``width`` elements: ``planes = ((heads, width), ...)``.  Keys and values of ``kv_heads`` heads of
    ``head_dim`` are two equal planes, which is what ``kv_heads`` / ``head_dim`` alone mean; one latent vector per token
    would be a single plane, keys and values of different widths two unequal ones.
    kind "state": one tensor of ``state_shape`` per request (always 32-bit).
    kind "none": nothing.
    """

    kind: str = "none"
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    state_shape: tuple[int, ...] = ()
    planes: tuple[tuple[int, int], ...] = ()

    def page_planes(self) -> tuple[tuple[int, int], ...]:
        """The planes of a page: as given, or keys and values of ``kv_heads`` x ``head_dim``."""
        if self.planes:
            return tuple((int(h), int(w)) for h, w in self.planes)
        return ((self.kv_heads, self.head_dim), (self.kv_heads, self.head_dim)) if self.kind == "pages" else ()

    def uniform_planes(self) -> bool:
        planes = self.page_planes()
        return all(plane == planes[0] for plane in planes)

    def group_key(self) -> tuple:
        return (self.kind, self.page_planes(), self.window, self.state_shape)


@dataclass
class LayerCache:
    """The cache of one run of a layer, as its mixer sees it during a step."""

    need: CacheNeed
    writes: bool = True
    pages: torch.Tensor | None = None        # equal planes: [num_pages, planes, heads, page_size, width] (keys and values: planes = 2)
    block_table: torch.Tensor | None = None  # int32 [requests in step, width], -1 where no page
    page_size: int = 0
    state: torch.Tensor | None = None        # [slots, *state_shape] float32
    plane_pages: tuple = ()                  # unequal planes: one [num_pages, heads, page_size, width] tensor per plane


class Workspace:
    """Named activation buffers of fixed address, sized once for the largest step.

    A buffer never moves and never grows: a captured CUDA graph keeps the address it saw, so a step of more rows than
    ``max_tokens`` is refused instead of being given a new buffer."""

    def __init__(self, device: torch.device, max_tokens: int):
        self.device = device
        self.max_tokens = max_tokens
        self._buffers: dict[tuple, torch.Tensor] = {}

    def get(self, name: str, rows: int, width: int, dtype: torch.dtype) -> torch.Tensor:
        if rows > self.max_tokens:
            raise BatchError(f"a step of {rows} rows does not fit the workspace of {self.max_tokens} (max_batch_tokens)")
        key = (name, width, dtype)
        buffer = self._buffers.get(key)
        if buffer is None:
            buffer = torch.empty((self.max_tokens, width), dtype=dtype, device=self.device)
            self._buffers[key] = buffer
        return buffer[:rows]


@dataclass
class Runtime:
    """Where and in which precision a model runs."""

    dtype: torch.dtype
    device: torch.device
    workspace: Workspace
    options: dict = field(default_factory=dict)


class Part:
    category = ""
    # True: forward launches kernels only and reads nothing of the step on the host (no ``ctx.host_*`` list, no ``.item()``),
    # so a step through it can be captured as a CUDA graph and replayed with other tokens.  A model is captured only if every
    # part of it says so; a part that says nothing runs kernel by kernel.
    capturable = False

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        return []

    def __init__(self, spec: PartSpec, prefix: str, weights, runtime: Runtime):
        self.spec = spec
        self.prefix = prefix
        self.runtime = runtime


def capturable(part) -> bool:
    """Whether the part and every part it holds can be captured (see ``Part.capturable``)."""
    if not part.capturable:
        return False
    return all(capturable(value) for value in vars(part).values() if isinstance(value, Part))


class Norm(Part):
    category = "norm"
    supports_lazy = False   # True: forward(..., lazy=True) may return an ops.LazyNorm for a product to apply

    def forward(self, residual, delta=None, rows=None):
        raise NotImplementedError


class PositionEncoding(Part):
    category = "position"

    def rotary_table(self):
        return None

    def apply(self, qkv, ctx, q_heads: int, kv_heads: int, head_dim: int) -> None:
        raise NotImplementedError


class Mixer(Part):
    category = "mixer"
    # A mixer (or feed-forward) that sets these takes more work into its own kernels when the block offers it:
    accepts_lazy_norm = False      # forward may receive an ops.LazyNorm in the place of the normalised tensor
    fuses_residual_add = False     # forward(..., accumulate_into=residual) adds its output there and returns None
    prepares_next_norm = False     # with accumulate_into it also takes prepare=<ops.LazyNorm of the norm that follows>

    def adds_to_residual(self, rows: int) -> bool:
        """Whether, with ``fuses_residual_add``, a step of this many rows beyond the fused row limit can still add in its last kernel."""
        return False

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        return CacheNeed()

    def forward(self, x, ctx, cache: LayerCache):
        raise NotImplementedError


class FeedForward(Part):
    category = "feed_forward"
    accepts_lazy_norm = False
    fuses_residual_add = False
    prepares_next_norm = False

    def adds_to_residual(self, rows: int) -> bool:
        return False

    def forward(self, x, ctx):
        raise NotImplementedError


class Block(Part):
    category = "block"
    accepts_next_norm = False      # forward(..., next_norm=<Norm>) : the norm that will read this block's result, if known
    first_norm = None              # the norm that reads this block's input first, if it has one: what the block before is told as ``next_norm``

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        return CacheNeed()

    def forward(self, residual, delta, ctx, cache: LayerCache):
        raise NotImplementedError


def norm_then_part(norm, part, residual, pending, fused: bool, next_norm, *args):
    """``part(norm(residual + pending))`` for a block of any kind, with what the small-step kernels can take over taken over.

    A block that arranges its parts differently (two parts from one norm, a norm after the part, ...) calls this once per
    (norm, part) pair and gets the decode fusions without knowing them: with few rows (``fused``: ``rows <=
    ops.fused_rows_limit(...)``) a part that ``accepts_lazy_norm`` applies the norm inside its first product, one that
    ``fuses_residual_add`` adds its output into ``residual`` itself, and one that ``prepares_next_norm`` leaves the input of
    ``next_norm`` (the norm that will read the residual next, or None) ready.  A part that declares none of this is handed the
    normalised tensor and its output is returned.

    ``pending``: None, an output not yet added to the residual, or an ``ops.LazyNorm`` that the product before left prepared
    (the residual is complete then).  ``args``: what the part's ``forward`` takes after ``x`` (``ctx``, and ``cache`` for a mixer).
    Returns what is pending after the part: None (the residual is complete), the part's output, or the prepared lazy norm."""
    from .. import ops

    lazily = fused and part.accepts_lazy_norm and norm.supports_lazy   # a norm that says nothing of laziness is never asked for it
    if isinstance(pending, ops.LazyNorm):
        if lazily and pending.weight is norm.weight and pending.eps == norm.eps:
            x = pending
        else:
            x = norm.forward(residual, None, lazy=True) if lazily else norm.forward(residual, None)
    elif lazily:
        x = norm.forward(residual, pending, lazy=True)
    else:
        x = norm.forward(residual, pending)
    if not fused and part.fuses_residual_add and part.adds_to_residual(residual.shape[0]):
        return part.forward(x, *args, accumulate_into=residual)   # many rows: the add happens in the last product's epilogue
    if fused and part.fuses_residual_add:
        if part.prepares_next_norm and next_norm is not None and next_norm.supports_lazy:
            following = next_norm.forward(residual, None, lazy=True)   # of the residual as it will be when the part is done
            part.forward(x, *args, accumulate_into=residual, prepare=following)
            return following
        return part.forward(x, *args, accumulate_into=residual)
    return part.forward(x, *args)


# --- registry of part classes -------------------------------------------------------------
_PARTS: dict[tuple[str, str], type] = {}
CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")


def register_part(category: str, kind: str, cls: type, *, replace: bool = False) -> None:
    if category not in CATEGORIES:
        raise ConfigError(f"unknown part category {category!r}")
    if (category, kind) in _PARTS and not replace:
        raise ConfigError(f"{category} part {kind!r} is already registered")
    _PARTS[(category, kind)] = cls


def unregister_part(category: str, kind: str) -> None:
    _PARTS.pop((category, kind), None)


def part_class(category: str, spec: PartSpec) -> type:
    try:
        return _PARTS[(category, spec.kind)]
    except KeyError:
        known = sorted(kind for cat, kind in _PARTS if cat == category)
        raise ConfigError(f"no {category} part of kind {spec.kind!r}; known: {known}") from None


def build_part(category: str, spec: PartSpec, prefix: str, weights, runtime: Runtime):
    return part_class(category, spec)(spec, prefix, weights, runtime)
