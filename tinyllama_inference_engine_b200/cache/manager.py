"""The cache manager: pages of keys and values, block tables, and per-request state slots.

What a model keeps between steps is declared by its mixers as ``CacheNeed``s, one per
cache stream of the model's order list.  Streams with the same need form a *group*:

* a **page group** (all keys, or a window of them) owns a page pool and, per request,
  a block table from logical page (position // page_size) to physical page.  One page
  id covers every stream of the group and every *plane* of a page (``CacheNeed.page_planes``:
  keys and values are two equal planes).  Equal planes share one device tensor
  ``[stream, page, plane, head, slot, width]``; unequal ones get a tensor each,
  ``[stream, page, head, slot, width]``.  Groups with different needs have pools of their own.  Pages go back to the pool when the request ends, and, in a
  window group, as soon as every later query is past them; they are handed out again
  without being cleared (positions beyond a request's length are never read).
* a **state group** holds one tensor of fixed size per request *slot* and stream,
  ``[stream, slot, *state_shape]`` in 32-bit, zeroed when a request is admitted.

The reference reserves a whole 512-token region per request and clears it on release
(app/server.cpp:96-128, src/cuda/model.cu:301-321); its only per-request state is
``next_positions[slot]`` (src/cuda/model.cu:51), which is ``computed`` here.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..errors import BatchError, EngineError, OutOfPages
from ..parts.base import CacheNeed, LayerCache
from .page_pool import PagePool


@dataclass
class RequestRecord:
    """The fixed-size record of a live request."""

    request_id: object
    slot: int
    computed: int = 0                                  # tokens whose cache entries are written
    tables: dict = field(default_factory=dict)         # group index -> list of page ids (-1 = given back)


class PageGroup:
    def __init__(self, index: int, need: CacheNeed, streams: list[int], page_size: int, num_pages: int):
        self.index = index
        self.need = need
        self.streams = streams
        self.page_size = page_size
        self.pool = PagePool(num_pages)
        self.tensor: torch.Tensor | None = None          # equal planes
        self.plane_tensors: list[torch.Tensor] = []       # unequal planes

    def tensors(self) -> list:
        return [self.tensor] if self.tensor is not None else list(self.plane_tensors)

    def pages_for(self, record: RequestRecord, new_total: int) -> int:
        """How many new pages positions < new_total need beyond the request's table."""
        table = record.tables.get(self.index, [])
        return max(0, -(-new_total // self.page_size) - len(table))

    def first_needed_page(self, computed: int) -> int:
        """Lowest logical page any query at position >= computed can still read."""
        if self.need.window <= 0:
            return 0
        return max(0, computed - self.need.window + 1) // self.page_size


class StateGroup:
    def __init__(self, index: int, need: CacheNeed, streams: list[int]):
        self.index = index
        self.need = need
        self.streams = streams
        self.tensor: torch.Tensor | None = None


class CacheManager:
    def __init__(self, needs: dict[int, CacheNeed], page_size: int, num_pages: int, max_requests: int,
                 max_positions: int, dtype: torch.dtype = torch.float32, device: torch.device | str | None = None,
                 poison_freed_pages: bool = False):
        self.page_size = page_size
        self.max_requests = max_requests
        self.table_width = -(-max_positions // page_size)
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else None
        self.poison = poison_freed_pages
        self.page_groups: list[PageGroup] = []
        self.state_groups: list[StateGroup] = []
        self.stream_group: dict[int, tuple[str, int, int]] = {}  # stream -> (kind, group index, index in group)
        by_key: dict[tuple, list[int]] = {}
        for stream in sorted(needs):
            by_key.setdefault(needs[stream].group_key(), []).append(stream)
        for key, streams in by_key.items():
            need = needs[streams[0]]
            if need.kind == "pages":
                group = PageGroup(len(self.page_groups), need, streams, page_size, num_pages)
                self.page_groups.append(group)
            elif need.kind == "state":
                group = StateGroup(len(self.state_groups), need, streams)
                self.state_groups.append(group)
            elif need.kind == "none":
                for stream in streams:
                    self.stream_group[stream] = ("none", 0, 0)
                continue
            else:
                raise EngineError(f"unknown cache need kind {need.kind!r}", code="invalid_argument")
            for position, stream in enumerate(streams):
                self.stream_group[stream] = (need.kind, group.index, position)
        self.needs = dict(needs)
        self._has_windows = any(group.need.window > 0 for group in self.page_groups)
        self.records: dict[object, RequestRecord] = {}
        self._free_slots = list(range(max_requests - 1, -1, -1))
        if self.device is not None:
            self._allocate_tensors()

    # --- device memory ------------------------------------------------------------------
    def _allocate_tensors(self) -> None:
        for group in self.page_groups:
            planes = group.need.page_planes()
            streams, pages = len(group.streams), group.pool.num_pages
            if group.need.uniform_planes():
                heads, width = planes[0]
                group.tensor = torch.zeros((streams, pages, len(planes), heads, self.page_size, width), dtype=self.dtype, device=self.device)
            else:
                group.plane_tensors = [torch.zeros((streams, pages, heads, self.page_size, width), dtype=self.dtype, device=self.device) for heads, width in planes]
            if self.poison:
                for tensor in group.tensors():
                    tensor.fill_(float("nan"))
        for group in self.state_groups:
            shape = (len(group.streams), self.max_requests, *group.need.state_shape)
            group.tensor = torch.zeros(shape, dtype=torch.float32, device=self.device)

    def cache_bytes(self) -> int:
        total = 0
        for group in self.page_groups:
            total += sum(tensor.numel() * tensor.element_size() for tensor in group.tensors())
        for group in self.state_groups:
            if group.tensor is not None:
                total += group.tensor.numel() * group.tensor.element_size()
        return total

    # --- requests -------------------------------------------------------------------------
    def has(self, request_id: object) -> bool:
        return request_id in self.records

    def computed(self, request_id: object) -> int:
        return self.records[request_id].computed

    def admit(self, request_id: object) -> RequestRecord:
        if request_id in self.records:
            raise BatchError(f"request {request_id!r} is already live")
        if not self._free_slots:
            raise OutOfPages(f"all {self.max_requests} request slots are taken")
        record = RequestRecord(request_id, self._free_slots.pop())
        self.records[request_id] = record
        for group in self.state_groups:
            if group.tensor is not None:
                group.tensor[:, record.slot].zero_()
        return record

    def can_admit(self) -> bool:
        return bool(self._free_slots)

    def pages_needed(self, request_id: object | None, new_total: int) -> list[int]:
        """New pages per page group for the request to hold positions < new_total."""
        record = self.records.get(request_id) if request_id is not None else None
        pages = -(-new_total // self.page_size)
        if record is None:
            return [pages] * len(self.page_groups)
        tables = record.tables
        return [max(0, pages - len(tables.get(group.index, ()))) for group in self.page_groups]

    def can_reserve(self, wanted: list[tuple[object | None, int]]) -> bool:
        """Whether all (request, new_total) pairs can get their pages at once."""
        totals = [0] * len(self.page_groups)
        for request_id, new_total in wanted:
            for index, count in enumerate(self.pages_needed(request_id, new_total)):
                totals[index] += count
        return all(total <= group.pool.free_count for total, group in zip(totals, self.page_groups))

    def reserve(self, request_id: object, new_total: int) -> None:
        """Pages for positions < new_total in every group, or OutOfPages with nothing taken."""
        record = self.records[request_id]
        counts = [group.pages_for(record, new_total) for group in self.page_groups]
        for group, count in zip(self.page_groups, counts):
            if count > group.pool.free_count:
                raise OutOfPages(
                    f"request {request_id!r} needs {count} more pages in cache group {group.index} "
                    f"(window {group.need.window or 'none'}), {group.pool.free_count} are free"
                )
        for group, count in zip(self.page_groups, counts):
            record.tables.setdefault(group.index, []).extend(group.pool.allocate(count, request_id))

    def advance(self, request_id: object, new_total: int) -> None:
        """The step wrote the cache up to ``new_total``; give back what a window has passed."""
        record = self.records[request_id]
        if new_total < record.computed:
            raise BatchError(f"request {request_id!r} cannot go back from {record.computed} to {new_total}")
        record.computed = new_total
        if not self._has_windows:
            return
        for group in self.page_groups:
            table = record.tables.get(group.index, [])
            passed = [i for i in range(min(group.first_needed_page(new_total), len(table))) if table[i] >= 0]
            if passed:
                pages = [table[i] for i in passed]
                self._give_back(group, pages, request_id)
                for i in passed:
                    table[i] = -1

    def release(self, request_id: object) -> None:
        """The request has ended: all its pages and its slot are free again."""
        record = self.records.pop(request_id)
        for group in self.page_groups:
            pages = [p for p in record.tables.get(group.index, []) if p >= 0]
            self._give_back(group, pages, request_id)
        self._free_slots.append(record.slot)

    def _give_back(self, group: PageGroup, pages: list[int], owner: object) -> None:
        if not pages:
            return
        group.pool.free(pages, owner)
        if self.poison:
            for tensor in group.tensors():
                tensor[:, torch.tensor(pages, device=tensor.device)] = float("nan")

    # --- what a step needs ----------------------------------------------------------------
    def block_table_rows(self, group: PageGroup, request_ids: list[object]) -> list[list[int]]:
        rows = []
        for request_id in request_ids:
            table = self.records[request_id].tables.get(group.index, [])
            if len(table) > self.table_width:
                raise BatchError(f"request {request_id!r} holds more pages than the block table is wide")
            rows.append(table + [-1] * (self.table_width - len(table)))
        return rows

    def layer_caches(self, block_tables: list[torch.Tensor]) -> dict[int, LayerCache]:
        """A LayerCache per cache stream, given this step's block tables (one per page group)."""
        caches: dict[int, LayerCache] = {}
        for stream, (kind, group_index, position) in self.stream_group.items():
            need = self.needs[stream]
            if kind == "pages":
                group = self.page_groups[group_index]
                caches[stream] = LayerCache(need, True, None if group.tensor is None else group.tensor[position], block_tables[group_index], self.page_size, None,
                                            tuple(tensor[position] for tensor in group.plane_tensors))
            elif kind == "state":
                group = self.state_groups[group_index]
                caches[stream] = LayerCache(need, True, None, None, 0, group.tensor[position])
            else:
                caches[stream] = LayerCache(need, True)
        return caches

    # --- accounting -----------------------------------------------------------------------
    def free_pages(self) -> list[int]:
        return [group.pool.free_count for group in self.page_groups]

    def max_total(self, request_id: object | None, free: list[int]) -> int:
        """The most tokens the request could hold if it got ``free[g]`` more pages in every group g."""
        record = self.records.get(request_id) if request_id is not None else None
        best = 1 << 60
        for group in self.page_groups:
            held = len(record.tables.get(group.index, [])) if record is not None else 0
            best = min(best, (held + free[group.index]) * self.page_size)
        return best

    def total_pages(self) -> list[int]:
        return [group.pool.num_pages for group in self.page_groups]

    def release_request(self, request_id: object) -> None:
        """``release`` that tolerates a request which never ran (nothing to give back)."""
        if request_id in self.records:
            self.release(request_id)

    def stats(self) -> dict:
        return {
            "live_requests": len(self.records),
            "free_slots": len(self._free_slots),
            "groups": [
                {"window": g.need.window, "streams": len(g.streams), "pages": g.pool.num_pages, "free": g.pool.free_count,
                 "allocations": g.pool.allocations, "reuses": g.pool.reuses}
                for g in self.page_groups
            ],
        }

    def check(self) -> None:
        """No page lost, none held twice, every held page in exactly one live table."""
        for group in self.page_groups:
            group.pool.check()
            held: dict[int, object] = {}
            for record in self.records.values():
                for page in record.tables.get(group.index, []):
                    if page < 0:
                        continue
                    if page in held:
                        raise EngineError(f"page {page} is in the tables of {held[page]!r} and {record.request_id!r}", code="out_of_bounds")
                    held[page] = record.request_id
                    if group.pool.owner_of(page) != record.request_id:
                        raise EngineError(f"page {page} is in a table of {record.request_id!r} but owned by {group.pool.owner_of(page)!r}", code="out_of_bounds")
            if len(held) != group.pool.used_count:
                raise EngineError(f"group {group.index}: {group.pool.used_count} pages are taken but tables hold {len(held)}", code="out_of_bounds")
        slots = [r.slot for r in self.records.values()] + self._free_slots
        if sorted(slots) != list(range(self.max_requests)):
            raise EngineError("request slots are lost or held twice", code="out_of_bounds")
