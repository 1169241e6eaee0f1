"""The step function: run a batch of (request, its next tokens) from the cache, return wanted logits.

``ModelRunner`` owns the model, the cache manager and nothing else.  ``step`` takes
any mixture of prompt portions and single decoded tokens, cut anywhere; it runs only
the tokens it is given, as one batch, and returns the logits at the wanted places.
The reference's counterpart takes exactly one token per request and returns logits for
every row (src/cuda/model.cu:531-725).
"""
from __future__ import annotations

from pathlib import Path

import torch

from ..cache import CacheManager
from ..config import EngineConfig, load_model_config
from ..errors import BatchError, KernelError
from ..models import DecoderModel, expected_tensors
from ..parts.base import Runtime, Workspace
from ..weights import WeightStore
from .batch import StepContext, StepEntry, lay_out_step, pack_step, step_shape
from .timing import StepClock, StepTimings

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}
STEP_GRAPH_AFTER_USES = 2    # a step shape is captured when it comes up the second time
MAX_STEP_GRAPHS = 32         # captured shapes kept (least recently used goes first)


class GraphedStep:
    """One step shape: its description's buffer of fixed address and, from its second use on, the CUDA graph of its kernels."""

    def __init__(self):
        self.uses = 0
        self.host: torch.Tensor | None = None
        self.device: torch.Tensor | None = None
        self.graph: torch.cuda.CUDAGraph | None = None
        self.logits: torch.Tensor | None = None

    def run(self, runner: "ModelRunner", entries, firsts, slots, table_rows) -> torch.Tensor | None:
        if self.host is None:
            words = len(lay_out_step(entries, firsts, slots, table_rows)["flat"])
            self.host = torch.zeros(words, dtype=torch.int32).pin_memory()
            self.device = torch.zeros(words, dtype=torch.int32, device=runner.device)
        ctx = pack_step(entries, firsts, slots, table_rows, runner.device, into=(self.host, self.device))
        # launch shapes chosen from the context length must hold for every later step of this shape
        ctx.max_seq_len = runner.spec.max_positions
        if self.graph is not None:
            self.graph.replay()
            return None if self.logits is None else self.logits.clone()   # the graph's own memory is written again by the next replay
        # This use runs kernel by kernel (with the settings the capture will have, so that every library and buffer it needs
        # exists), then the same launches are recorded for the uses to come.
        logits = runner.run(ctx)
        graph = torch.cuda.CUDAGraph()
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            graph.capture_begin()
            try:
                self.logits = runner.run(ctx)
            finally:
                graph.capture_end()
        torch.cuda.current_stream().wait_stream(stream)
        self.graph = graph
        return logits


class ModelRunner:
    def __init__(self, model_dir: str | Path, engine_config: EngineConfig | None = None):
        self.engine_config = engine_config or EngineConfig()
        self.device = torch.device(self.engine_config.device)
        if self.device.type == "cuda" and not torch.cuda.is_available():
            raise KernelError("no CUDA device is visible; this engine has no CPU path")
        self.architecture, self.model_config = load_model_config(model_dir)
        self.spec = self.architecture.build_spec(self.model_config)
        self.dtype = _TORCH_DTYPES[self.engine_config.dtype]
        if self.engine_config.weights_sha256:
            from ..weights.integrity import verify_weights

            verify_weights(model_dir, self.engine_config.weights_sha256)
        weights = WeightStore.load(model_dir, expected_tensors(self.spec), self.device)
        workspace = Workspace(self.device, self.engine_config.max_batch_tokens)
        self.runtime = Runtime(self.dtype, self.device, workspace, {"engine": self.engine_config})
        self.model = DecoderModel(self.spec, weights, self.runtime)
        del weights
        self.cache = CacheManager(
            self.model.cache_needs, self.engine_config.page_size, self.engine_config.num_pages,
            self.engine_config.max_requests, self.spec.max_positions, self.dtype, self.device,
            poison_freed_pages=self.engine_config.poison_freed_pages,
        )
        self.steps = 0
        self.tokens_run = 0
        self._step_graphs: dict[tuple, GraphedStep] = {}

    # --- the step --------------------------------------------------------------------------
    def validate(self, entries: list[StepEntry]) -> list[int]:
        """Check a batch without changing anything; returns each entry's first position."""
        if not entries:
            raise BatchError("a step needs at least one entry")
        seen = set()
        firsts = []
        vocab = self.spec.vocab_size
        new_requests = 0
        for entry in entries:
            if entry.request_id in seen:
                raise BatchError(f"request {entry.request_id!r} appears twice in one step")
            seen.add(entry.request_id)
            if not entry.tokens:
                raise BatchError(f"request {entry.request_id!r} brings no tokens")
            if min(entry.tokens) < 0 or max(entry.tokens) >= vocab:
                token = next(token for token in entry.tokens if not 0 <= token < vocab)
                raise BatchError(f"token {token} of request {entry.request_id!r} is outside the vocabulary of {vocab}")
            for place in entry.want:
                if not 0 <= place < len(entry.tokens):
                    raise BatchError(f"request {entry.request_id!r} wants place {place} among {len(entry.tokens)} tokens")
            first = self.cache.computed(entry.request_id) if self.cache.has(entry.request_id) else 0
            new_requests += not self.cache.has(entry.request_id)
            if first + len(entry.tokens) > self.spec.max_positions:
                raise BatchError(
                    f"request {entry.request_id!r} would reach {first + len(entry.tokens)} tokens; the model's context is {self.spec.max_positions}"
                )
            firsts.append(first)
        total = sum(len(entry.tokens) for entry in entries)
        if total > self.engine_config.max_batch_tokens:
            raise BatchError(f"the step brings {total} tokens; max_batch_tokens is {self.engine_config.max_batch_tokens}")
        if len(self.cache.records) + new_requests > self.cache.max_requests:
            raise BatchError(f"more than {self.cache.max_requests} live requests")
        return firsts

    def step(self, entries: list[StepEntry], timings: StepTimings | None = None, trace: dict | None = None) -> torch.Tensor | None:
        """Run the entries as one batch; returns 32-bit logits [wanted, vocab] (None if nothing is wanted).

        ``timings``: filled with what the step cost (the call then waits for the device).  ``trace``: filled with the hidden
        state after every run of a layer, ``trace["layer<i>.output"]`` [rows, hidden] in 32-bit, as the reference's traced
        forward keeps them (src/model.cpp:98-100, 200-206), so that a wrong logit can be followed back to its layer."""
        clock = StepClock(self.device, timings is not None)
        firsts = self.validate(entries)
        wanted = [(e.request_id if self.cache.has(e.request_id) else None, f + len(e.tokens)) for e, f in zip(entries, firsts)]
        if not self.cache.can_reserve(wanted):
            from ..errors import OutOfPages

            raise OutOfPages(f"the step needs more cache pages than are free ({self.cache.free_pages()} free)")
        slots = []
        for entry, first in zip(entries, firsts):
            if not self.cache.has(entry.request_id):
                self.cache.admit(entry.request_id)
            self.cache.reserve(entry.request_id, first + len(entry.tokens))
            slots.append(self.cache.records[entry.request_id].slot)
        ids = [e.request_id for e in entries]
        table_rows = [self.cache.block_table_rows(group, ids) for group in self.cache.page_groups]
        graphed = self._graphed_step(entries) if timings is None and trace is None else None
        if graphed is not None:
            logits = graphed.run(self, entries, firsts, slots, table_rows)
        else:
            ctx = pack_step(entries, firsts, slots, table_rows, self.device)
            clock.mark()
            logits = self.run(ctx, trace)
            clock.mark()
        for entry, first in zip(entries, firsts):
            self.cache.advance(entry.request_id, first + len(entry.tokens))
        self.steps += 1
        self.tokens_run += sum(len(entry.tokens) for entry in entries)
        clock.finish(timings, ("transfer", "compute"))
        return logits

    def _graphed_step(self, entries: list[StepEntry]):
        """The captured form of steps of this shape, once the shape has come up often enough to be worth capturing (else None).

        A prompt portion of a few hundred tokens is some 160 kernels of a few microseconds each: launched one by one the host
        needs 2.8 ms for them whatever the GPU takes (0.6 to 2 ms).  A shape that repeats is captured the second time it runs
        and replayed from then on; the step's description (tokens, positions, block tables, work lists) lives in a buffer of
        fixed address that every replay refreshes with one copy."""
        if not (self.engine_config.use_cuda_graphs and self.device.type == "cuda" and self.model.capturable):
            return None   # some part reads the step on the host: kernel by kernel
        shape = step_shape(entries)
        slot = self._step_graphs.get(shape)
        if slot is None:
            if len(self._step_graphs) >= MAX_STEP_GRAPHS:
                self._step_graphs.pop(next(iter(self._step_graphs)))   # the shape seen longest ago
            slot = self._step_graphs[shape] = GraphedStep()
        else:
            self._step_graphs[shape] = self._step_graphs.pop(shape)   # most recently used last
        slot.uses += 1
        return slot if slot.uses >= STEP_GRAPH_AFTER_USES else None

    def run(self, ctx: StepContext, trace: dict | None = None) -> torch.Tensor | None:
        caches = self.cache.layer_caches(ctx.block_tables)
        return self.model.forward(ctx, caches, trace)

    def finish(self, request_id: object) -> None:
        """The request has ended; what it holds is given back."""
        if self.cache.has(request_id):
            self.cache.release(request_id)
