"""A set of requests decoding one token per step, replayed as one CUDA graph.

A decode step of this model is some hundred small kernels; launched one by one the
host cannot keep up with a B200 (the reference issues ~332 launches per token,
src/cuda/model.cu:406-475).  A session keeps the step's metadata (tokens, positions,
block tables, sampling options) in device buffers of fixed address, captures
forward + sampling + "move on by one position" once, and replays it.  Between
replays the host only reserves a page when a request crosses a page edge and copies
the changed block-table rows.  The graph's launch shapes depend on the number of
requests and on static limits only, never on the current lengths.
"""
from __future__ import annotations

import torch

from .. import ops
from ..errors import BatchError, KernelError
from .batch import decode_context, decode_layout

# A session runs its first steps kernel by kernel and is captured as a graph only when it is still in use after them:
# a batch that changes with every step (requests finishing one after another) would otherwise pay a capture, which costs
# as much as ten steps, for every size it passes through.
EAGER_STEPS_BEFORE_CAPTURE = 2


class DecodeSession:
    def __init__(self, runner, count: int, use_graph: bool = True, publish: bool = True):
        self.runner = runner
        self.publish = publish   # False: steps that stay on the device (nothing is written to host memory; read_tokens() copies)
        self.cache = runner.cache
        self.request_ids: list = []
        self.count = count
        device = runner.device
        width = self.cache.table_width
        groups = len(self.cache.page_groups)
        # one int32 buffer laid out as the packer lays a step out (engine.batch.decode_layout): host copy and device copy
        sizes = decode_layout(count, width, groups)
        self._host = torch.zeros(sum(sizes), dtype=torch.int32).pin_memory()
        self._device = torch.zeros(sum(sizes), dtype=torch.int32, device=device)
        self.ctx, offsets = decode_context(self._device, count, width, groups, runner.spec.max_positions, self.request_ids)
        self._offsets = offsets
        view = lambda buffer, i: buffer[offsets[i] : offsets[i + 1]]  # noqa: E731
        self.h_tokens, self.h_positions = view(self._host, 0), view(self._host, 1)
        self._np = self._host.numpy()                       # the same pinned memory, for cheap host writes
        self._d_tokens = self._device[:count]               # where the step's input ids lie on the device
        # The step's result also arrives by itself: the last kernel of a step writes the tokens, the device error word and the
        # step's number into this pinned memory over the bus, and read_tokens() polls the number instead of waiting for two
        # copies and the stream (some 25 us of every step with the host in the loop).
        self._mailbox = torch.zeros(count + 2, dtype=torch.int32).pin_memory()
        self._mail = self._mailbox.numpy()
        self._steps_done = torch.zeros(1, dtype=torch.int32, device=device)
        self._steps_issued = 0
        self._error_word = ops.error_flag(device)            # what kernels of this device report without a host in the loop
        self._capacity = [0] * count                        # tokens each request's pages hold (least over the groups)
        self.h_tables = [view(self._host, 8 + g).view(count, width) for g in range(groups)]
        view(self._host, 2).copy_(torch.arange(count))
        view(self._host, 3).copy_(torch.arange(count + 1))
        view(self._host, 7).copy_(torch.arange(count))
        self.d_tables = self.ctx.block_tables
        self.sampled = torch.zeros(count, dtype=torch.int32, device=device)
        self.temperature = torch.zeros(count, dtype=torch.float32, device=device)
        self.top_p = torch.ones(count, dtype=torch.float32, device=device)
        self.seeds = torch.zeros(count, dtype=torch.int64, device=device)
        self.counters = torch.zeros(count, dtype=torch.int64, device=device)
        self.positions = [0] * count      # host mirror: position of the token each request runs next
        self.use_graph = use_graph
        self._fresh = True
        self._loaded = False
        self._eager_steps = 0
        self.graph: torch.cuda.CUDAGraph | None = None
        self.logits: torch.Tensor | None = None
        self.kernels_per_step = 0          # kernels of this engine in one step (counted while warming up)
        self.library_calls_per_step = 0    # vendor-library matrix products in one step

    # --- loading -----------------------------------------------------------------------------
    def load(self, request_ids: list, tokens: list[int], params: list | None = None, draw_indices: list[int] | None = None) -> None:
        """Bind ``count`` live requests: each one's next token (at the position its cache has reached) and sampling options."""
        if len(request_ids) != self.count or len(set(request_ids)) != self.count:
            raise BatchError(f"this decode session holds exactly {self.count} different requests")
        self.request_ids = list(request_ids)
        self.ctx.request_ids = self.request_ids
        self._fresh = True
        slots = []
        for i, request_id in enumerate(self.request_ids):
            if not self.cache.has(request_id):
                raise BatchError(f"request {request_id!r} is not live; a decode session continues requests that were prefilled")
            self.positions[i] = self.cache.computed(request_id)
            slots.append(self.cache.records[request_id].slot)
        o = self._offsets
        self._np[o[0] : o[1]] = tokens
        self._np[o[1] : o[2]] = self.positions
        self._np[o[4] : o[5]] = [p + 1 for p in self.positions]   # seq_lens
        self._np[o[5] : o[6]] = self.positions                    # first_positions
        self._np[o[6] : o[7]] = slots
        self.ctx.host_state_slots = slots
        self._reserve_and_fill_tables()
        self._fresh = False
        self._loaded = True
        self._device.copy_(self._host, non_blocking=True)
        if params is not None:
            self.temperature.copy_(torch.tensor([p.temperature for p in params], dtype=torch.float32))
            self.top_p.copy_(torch.tensor([p.top_p for p in params], dtype=torch.float32))
            self.seeds.copy_(torch.tensor([p.seed for p in params], dtype=torch.int64))
            self.counters.copy_(torch.tensor(draw_indices or [0] * self.count, dtype=torch.int64))

    def _reserve_and_fill_tables(self) -> bool:
        """Pages for this step's positions; returns whether any block-table row changed."""
        changed = False
        page_size = self.cache.page_size
        for i, request_id in enumerate(self.request_ids):
            if self.positions[i] < self._capacity[i] and not self._fresh:
                continue  # the position lies in a page the request already holds
            self.cache.reserve(request_id, self.positions[i] + 1)
            record = self.cache.records[request_id]
            capacity = 1 << 60
            for g, group in enumerate(self.cache.page_groups):
                table = record.tables.get(group.index, [])
                capacity = min(capacity, len(table) * page_size)
                row = self.h_tables[g][i].numpy()
                row[:] = -1
                row[: len(table)] = table
            self._capacity[i] = capacity
            changed = True
        return changed

    # --- stepping ----------------------------------------------------------------------------
    def _body(self) -> None:
        if self.publish:
            # host in the loop: the step's input ids come from pinned host memory, by a copy that is part of the step (of its graph)
            self._d_tokens.copy_(self.h_tokens, non_blocking=True)
        caches = self.cache.layer_caches(self.d_tables)
        self.logits = self.runner.model.forward(self.ctx, caches)
        ops.sample(self.logits, self.temperature, self.top_p, self.seeds, self.counters, self.sampled)
        c = self.ctx
        if self.publish:
            ops.decode_advance(c.token_ids, self.sampled, c.positions, c.seq_lens, c.first_positions, self.counters, self._mailbox, self._steps_done)
        else:
            ops.decode_advance(c.token_ids, self.sampled, c.positions, c.seq_lens, c.first_positions, self.counters)

    def set_tokens(self, tokens: list[int]) -> None:
        """Host tokens in: the step's input ids come from pinned host memory."""
        self._np[: self.count] = tokens
        if not self.publish:
            self._d_tokens.copy_(self.h_tokens, non_blocking=True)

    def next_step_fits_its_pages(self) -> bool:
        """Whether every request's next position lies in a page it already holds (then the next step reserves nothing)."""
        capacity = self._capacity
        for i, position in enumerate(self.positions):
            if position >= capacity[i]:
                return False
        return not self._fresh

    def read_tokens(self) -> list[int]:
        """Host tokens out: the tokens the last step sampled, as its last kernel wrote them into pinned host memory."""
        if not self.publish:
            tokens = self.sampled.cpu()
            ops.check_device_errors(self.sampled.device)
            return tokens.tolist()
        mail, last, wanted = self._mail, self.count + 1, self._steps_issued
        stream = torch.cuda.current_stream()
        polls = 0
        while mail[last] != wanted:
            polls += 1
            if polls % 4096 == 0 and stream.query() and mail[last] != wanted:
                # the stream has nothing left to run and the number never came: a kernel of the step failed
                stream.synchronize()
                raise KernelError("a decode step ended without publishing its result")
        ops.raise_for_error_word(int(mail[self.count]), self._error_word.device)
        return mail[: self.count].tolist()

    def step(self) -> torch.Tensor:
        """One decode step for every request; returns the sampled tokens (device, int32).

        The tokens run are those on the device: the ones loaded, or the previous step's samples.
        """
        if not self._loaded:  # load() already reserved and copied the tables of its first step
            if self._reserve_and_fill_tables():
                o = self._offsets
                self._device[o[8] :].copy_(self._host[o[8] :], non_blocking=True)
        self._loaded = False
        if not self.use_graph or self.graph is None and self._eager_steps < EAGER_STEPS_BEFORE_CAPTURE:
            if self._eager_steps == 0:
                from ..ops import fast

                before, library_before = ops.launch_count, fast.library_gemm_calls
                self._body()
                self.kernels_per_step = ops.launch_count - before
                self.library_calls_per_step = fast.library_gemm_calls - library_before
            else:
                self._body()
            self._eager_steps += 1
        elif self.graph is None:
            # The steps run so far have made the workspaces and library handles, so the step can be captured as it is.
            # capture_begin / capture_end directly: the context manager of torch.cuda.graph also collects garbage and
            # empties the allocator's cache first, which can take longer than a hundred steps.
            self.graph = torch.cuda.CUDAGraph()
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                self.graph.capture_begin()
                try:
                    self._body()
                finally:
                    self.graph.capture_end()
            torch.cuda.current_stream().wait_stream(stream)
            # capture does not run anything: the step itself is the first replay
            self.graph.replay()
        else:
            self.graph.replay()
        self._steps_issued += 1
        advance = self.cache.advance
        for i, request_id in enumerate(self.request_ids):
            self.positions[i] += 1
            advance(request_id, self.positions[i])
        self.runner.steps += 1
        self.runner.tokens_run += self.count
        return self.sampled
