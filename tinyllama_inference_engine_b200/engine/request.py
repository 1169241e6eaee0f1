"""A generation request and its sampling options."""
from __future__ import annotations

from dataclasses import dataclass, field

from ..errors import EngineError


@dataclass
class SamplingParams:
    """Options of one request, with the reference's names and defaults (app/server.cpp:601-613).

    max_tokens   how many tokens to generate (the reference's default is 16).
    temperature  0 selects the largest logit (lowest id on ties); > 0 samples.
    top_p        keep the most probable tokens whose share reaches top_p (1 keeps all).
    seed         seed of the request's own random stream; draws do not depend on the batch.
    ignore_eos   the reference never stops at the end-of-sequence token (it runs exactly
                 max_tokens, app/server.cpp:468-470); False stops when ``eos_token_id`` is drawn.
    """

    max_tokens: int = 16
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int = 0
    ignore_eos: bool = True

    def __post_init__(self) -> None:
        if isinstance(self.max_tokens, bool) or not isinstance(self.max_tokens, int) or self.max_tokens < 1:
            raise EngineError("max_tokens must be an integer >= 1")
        if not self.temperature >= 0.0:
            raise EngineError("temperature must be >= 0")
        if not 0.0 < self.top_p <= 1.0:
            raise EngineError("top_p must be in (0, 1]")


WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Request:
    """State of a request between steps (app/server.cpp:43-94 without the serving fields)."""

    request_id: str
    prompt: list[int]
    params: SamplingParams
    arrival: int = 0
    state: str = WAITING
    generated: list[int] = field(default_factory=list)
    computed: int = 0            # tokens of prompt + generated whose cache entries exist
    preemptions: int = 0
    finish_reason: str | None = None   # "length", "stop", "cancelled"

    @property
    def tokens(self) -> list[int]:
        return self.prompt + self.generated

    def next_tokens(self, count: int) -> list[int]:
        """The ``count`` tokens after the ones already run."""
        start, split = self.computed, len(self.prompt)
        if start >= split:
            return self.generated[start - split : start - split + count]
        return (self.prompt[start : start + count] + self.generated[: max(0, start + count - split)])[:count]

    @property
    def total(self) -> int:
        return len(self.prompt) + len(self.generated)

    @property
    def remaining(self) -> int:
        """Tokens known but not yet run; the last of them yields the next token."""
        return len(self.prompt) + len(self.generated) - self.computed
