"""Continuous batching: which requests run in the next step, and with how many tokens each.

Policy, in the reference's spirit (app/server.cpp:360-408: decodes first from a rotating
cursor, then prefills, FIFO admission) but over tokens instead of rows:

1. running requests that only need one token (decode) come first, one token each,
   starting at a rotating cursor so that no request starves when the budget is short;
2. running requests still in their prompt get portions, in order of arrival, until
   the step's token budget (``max_batch_tokens``) is spent: a prompt is cut wherever
   the budget ends;
3. waiting requests are admitted in order of arrival while a request slot is free,
   the budget has room and their first portion's pages can be reserved.

When pages run out for a request that is already running, the request admitted last
is preempted: its pages are freed, it goes back to the front of the waiting queue and
later recomputes prompt + generated tokens from the start (greedy output is unchanged,
and sampled output too, since draws are numbered per request).  A request is never
preempted to admit a new one.  A request that cannot fit even alone fails at submission.

The scheduler decides; it runs nothing.  It sees the cache only through
``pages_needed`` / ``free_pages`` / ``can_admit``, so it is tested without a GPU.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..errors import EngineError
from .request import FINISHED, RUNNING, WAITING, Request


@dataclass
class ScheduledPortion:
    request: Request
    num_tokens: int
    pages: list[int] = field(default_factory=list)   # new pages per cache group this portion will take

    @property
    def samples(self) -> bool:
        """Whether this portion reaches the request's last known token, so its last row yields a new token."""
        return self.request.computed + self.num_tokens == self.request.total


class Scheduler:
    def __init__(self, cache, max_batch_tokens: int, max_requests: int, max_positions: int):
        self.cache = cache
        self.max_batch_tokens = max_batch_tokens
        self.max_requests = min(max_requests, cache.max_requests)
        self.max_positions = max_positions
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self._cursor = 0
        self._arrivals = 0
        self.preemptions = 0
        self.steps = 0

    # --- submission -----------------------------------------------------------------------
    def add(self, request: Request) -> None:
        if not request.prompt:
            raise EngineError("a request needs at least one prompt token")
        limit = len(request.prompt) + request.params.max_tokens
        if limit > self.max_positions:
            raise EngineError(f"prompt plus output exceeds context length ({limit} > {self.max_positions})", code="out_of_bounds")
        # the last generated token is never run, so limit - 1 positions are cached
        alone = self.cache.pages_needed(None, limit - 1)
        if any(need > pages for need, pages in zip(alone, self.cache.total_pages())):
            raise EngineError("the request does not fit the cache even alone", code="out_of_memory")
        request.arrival = self._arrivals
        self._arrivals += 1
        request.state = WAITING
        self.waiting.append(request)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # --- the decision -----------------------------------------------------------------------
    def schedule(self) -> list[ScheduledPortion]:
        """The portions of the next step.  May preempt (and so change the cache) but runs nothing."""
        budget = self.max_batch_tokens
        free = list(self.cache.free_pages())
        chosen: list[ScheduledPortion] = []

        def try_take(request: Request, tokens: int, live: bool) -> bool:
            need = self.cache.pages_needed(request.request_id if live else None, request.computed + tokens)
            if any(n > f for n, f in zip(need, free)):
                return False
            for i, n in enumerate(need):
                free[i] -= n
            chosen.append(ScheduledPortion(request, tokens, need))
            return True

        decodes, prefills = [], []
        for r in self.running:
            (decodes if r.remaining == 1 else prefills).append(r)
        prefills.sort(key=lambda r: r.arrival)
        if decodes:
            start = self._cursor % len(decodes)
            decodes = decodes[start:] + decodes[:start]
        taken_decodes = 0
        for request in decodes + prefills:
            while request.state == RUNNING and budget > 0:
                remaining = request.remaining
                tokens = min(remaining, budget)
                if try_take(request, tokens, live=True):
                    budget -= tokens
                    taken_decodes += remaining == 1
                    break
                room = self.cache.max_total(request.request_id, free) - request.computed
                if 1 <= room < tokens and try_take(request, room, live=True):
                    budget -= room   # a shorter portion fills the pages that are left
                    break
                # pages ran out: the request admitted last gives way (possibly this one)
                victim = max(self.running, key=lambda r: r.arrival)
                budget += self._preempt(victim, chosen, free)
        self._cursor += taken_decodes

        while self.waiting and budget > 0 and len(self.running) < self.max_requests:
            request = self.waiting[0]
            tokens = min(request.remaining, budget)
            if not try_take(request, tokens, live=False):
                break
            self.waiting.popleft()
            request.state = RUNNING
            self.running.append(request)
            budget -= tokens
        if not chosen and self.has_unfinished():
            raise EngineError("the scheduler cannot place any request: pages are held by nobody it can preempt", code="out_of_memory")
        self.steps += 1
        return chosen

    def _preempt(self, victim: Request, chosen: list[ScheduledPortion], free: list[int]) -> int:
        """Give back everything ``victim`` holds; it will recompute from its first token.  Returns budget regained."""
        regained = 0
        for portion in [p for p in chosen if p.request is victim]:
            chosen.remove(portion)
            regained += portion.num_tokens
            for i, n in enumerate(portion.pages):
                free[i] += n
        before = list(self.cache.free_pages())
        self.cache.release_request(victim.request_id)
        for i, after in enumerate(self.cache.free_pages()):
            free[i] += after - before[i]
        victim.computed = 0
        victim.state = WAITING
        victim.preemptions += 1
        self.preemptions += 1
        self.running.remove(victim)
        self.waiting.appendleft(victim)
        return regained

    # --- after a step -------------------------------------------------------------------------
    def finish(self, request: Request, reason: str) -> None:
        request.state = FINISHED
        request.finish_reason = reason
        if request in self.running:
            self.running.remove(request)
        elif request in self.waiting:
            self.waiting.remove(request)
        self.cache.release_request(request.request_id)
