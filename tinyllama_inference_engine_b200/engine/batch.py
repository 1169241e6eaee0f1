"""One step's batch: requests' next tokens, flattened, with everything a kernel needs to find the cache."""
from __future__ import annotations

from dataclasses import dataclass, field
from itertools import chain

import numpy as np
import torch


# --- per-step work lists -----------------------------------------------------------------------
# A kernel may want, beside the step's description, a list of work items that depends on how the step is cut (which runs of
# rows form a tile, in which order they are best run).  Whoever owns the kernel registers a function for it here; the packer
# calls every registered function once per step and ships the lists in the same buffer and the same copy as everything
# else.  The packer itself knows no kernel and no tile size.
@dataclass(frozen=True)
class StepPlan:
    name: str
    columns: int                                   # the list is int32 [n, columns]
    build: "callable"                              # (q_lens, first_positions, seq_starts) -> flat list of ints
    wanted: "callable" = lambda q_lens: True       # (q_lens) -> whether this step needs the list at all


_STEP_PLANS: dict[str, StepPlan] = {}


def register_step_plan(plan: StepPlan, *, replace: bool = False) -> None:
    if plan.name in _STEP_PLANS and not replace:
        raise ValueError(f"step plan {plan.name!r} is already registered")
    _STEP_PLANS[plan.name] = plan


def unregister_step_plan(name: str) -> None:
    _STEP_PLANS.pop(name, None)


@dataclass
class StepEntry:
    """The next tokens of one request and the places among them whose logits are wanted."""

    request_id: object
    tokens: list[int]
    want: list[int] = field(default_factory=list)


@dataclass
class StepContext:
    """Device-side description of a step (int32 tensors) plus the same numbers on the host.

    Rows of the step are the tokens of all entries, entry after entry.
      token_ids[T], positions[T]  each row's token and absolute position in its request
      token_seq[T]                which entry (request of this step) a row belongs to
      seq_starts[B + 1]           first row of every entry (cumulative lengths)
      seq_lens[B]                 tokens the request holds after this step
      first_positions[B]          position of the entry's first row
      state_slots[B]              the request's slot in per-request state tensors
      want_rows[W]                rows whose logits are returned, in entry and want order
      block_tables[g][B, width]   page ids of every entry in page group g (-1: none)
      plans[name][N, columns]     work lists registered with ``register_step_plan`` (see ``plan``)
    """

    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_seq: torch.Tensor
    seq_starts: torch.Tensor
    seq_lens: torch.Tensor
    first_positions: torch.Tensor
    state_slots: torch.Tensor
    want_rows: torch.Tensor | None
    block_tables: list[torch.Tensor]
    # host copies (plain lists) for parts written in Python and for kernel launch shapes
    request_ids: list
    host_q_lens: list[int]
    host_first_positions: list[int]
    host_state_slots: list[int]
    max_q_len: int
    max_seq_len: int
    wants_every_row_in_order: bool = False      # want_rows is 0, 1, ..., num_tokens - 1
    plans: dict = field(default_factory=dict)   # name -> int32 [n, columns] work list of a registered step plan

    @property
    def decode_only(self) -> bool:
        return self.max_q_len == 1

    def plan(self, name: str):
        """The work list ``name`` of this step, or None if nobody registered it or this step has no use for it."""
        return self.plans.get(name)


def lay_out_step(entries: list[StepEntry], first_positions: list[int], slots: list[int], table_rows: list[list[list[int]]]) -> dict:
    """The step as one flat array of int32 words and where its sections lie (host work only).

    Sections that have a word per token are made with numpy (a 2,048-token portion costs 0.1 ms so, 0.3 ms as Python lists)."""
    q_lens = [len(e.tokens) for e in entries]
    num_tokens, num_seqs = sum(q_lens), len(entries)
    lens = np.asarray(q_lens, dtype=np.int32)
    starts = np.zeros(num_seqs + 1, dtype=np.int32)
    np.cumsum(lens, out=starts[1:])
    seq_starts = starts.tolist()
    token_ids = np.fromiter(chain.from_iterable(e.tokens for e in entries), dtype=np.int32, count=num_tokens)
    shift = np.asarray(first_positions, dtype=np.int32) - starts[:-1]           # position of a row = its index + its entry's shift
    positions = np.arange(num_tokens, dtype=np.int32) + np.repeat(shift, lens)
    token_seq = np.repeat(np.arange(num_seqs, dtype=np.int32), lens)
    want_rows = [start + w for start, entry in zip(seq_starts, entries) for w in entry.want]
    seq_lens = [f + n for f, n in zip(first_positions, q_lens)]
    plans = [plan for plan in _STEP_PLANS.values() if plan.wanted(q_lens)]
    sections = [token_ids, positions, token_seq, starts, seq_lens, first_positions, slots, want_rows]
    sections += [plan.build(q_lens, first_positions, seq_starts) for plan in plans]
    offsets, words = [], 0
    for section in sections:
        offsets.append((words, len(section)))
        words += len(section)
    table_offsets = []
    for rows in table_rows:
        width = len(rows[0]) if rows else 0
        table_offsets.append((words, num_seqs, width))
        sections.append(np.asarray(rows, dtype=np.int32).reshape(-1))
        words += num_seqs * width
    flat = np.concatenate([np.asarray(section, dtype=np.int32) for section in sections])
    return {"flat": flat, "offsets": offsets, "table_offsets": table_offsets, "plans": plans, "q_lens": q_lens, "seq_lens": seq_lens,
            "num_tokens": num_tokens, "num_seqs": num_seqs, "want_rows": want_rows}


def pack_step(entries: list[StepEntry], first_positions: list[int], slots: list[int], table_rows: list[list[list[int]]],
              device: torch.device, into: tuple | None = None) -> StepContext:
    """Flatten the entries into one int32 buffer, copy it once, and slice the views.

    ``into``: (pinned host tensor, device tensor) of fixed address to write and copy into, for a step whose kernels were captured
    in a CUDA graph and read their description from there; they must be at least as long as the step's layout."""
    layout = lay_out_step(entries, first_positions, slots, table_rows)
    flat, offsets, table_offsets, plans = layout["flat"], layout["offsets"], layout["table_offsets"], layout["plans"]
    if into is None:
        host = torch.from_numpy(flat)
        if device.type == "cuda":
            host = host.pin_memory()
        buffer = host.to(device, non_blocking=True)
    else:
        host, buffer = into
        host.numpy()[: len(flat)] = flat
        buffer[: len(flat)].copy_(host[: len(flat)], non_blocking=True)
    views = [buffer[o : o + n] for o, n in offsets]
    tables = [buffer[o : o + b * w].view(b, w) for o, b, w in table_offsets]
    want_rows, num_tokens = layout["want_rows"], layout["num_tokens"]
    return StepContext(
        num_tokens=num_tokens, num_seqs=layout["num_seqs"],
        token_ids=views[0], positions=views[1], token_seq=views[2], seq_starts=views[3], seq_lens=views[4],
        first_positions=views[5], state_slots=views[6], want_rows=views[7] if want_rows else None,
        block_tables=tables, request_ids=[e.request_id for e in entries], host_q_lens=layout["q_lens"],
        host_first_positions=list(first_positions), host_state_slots=list(slots),
        max_q_len=max(layout["q_lens"]), max_seq_len=max(layout["seq_lens"]), wants_every_row_in_order=len(want_rows) == num_tokens and want_rows == list(range(num_tokens)),
        plans={plan.name: views[8 + i].view(-1, plan.columns) for i, plan in enumerate(plans)},
    )


def step_shape(entries: list[StepEntry]) -> tuple:
    """What of a step decides its kernels' launch shapes and its buffer's layout: every entry's number of tokens and of wanted
    places (and whether all rows are wanted in order).  Everything else about it is data the kernels read on the device."""
    in_order = all(entry.want == list(range(len(entry.tokens))) for entry in entries)
    return tuple((len(entry.tokens), len(entry.want)) for entry in entries) + (in_order,)


def decode_context(buffer: torch.Tensor, count: int, table_width: int, groups: int, max_positions: int, request_ids: list) -> tuple["StepContext", list]:
    """The context of a step of ``count`` single decoded tokens over a device buffer of fixed address (a decode session's), laid
    out as ``pack_step`` lays a step out: [tokens | positions | token_seq | seq_starts | seq_lens | first_positions | slots | want |
    tables...].  Returns the context and the section offsets.  ``max_seq_len`` is the longest context a request can reach, so
    that launch shapes chosen from it hold for every later step of the session."""
    sizes = decode_layout(count, table_width, groups)
    offsets = [0]
    for size in sizes:
        offsets.append(offsets[-1] + size)
    view = [buffer[offsets[i] : offsets[i + 1]] for i in range(len(sizes))]
    tables = [view[8 + g].view(count, table_width) for g in range(groups)]
    ctx = StepContext(
        num_tokens=count, num_seqs=count, token_ids=view[0], positions=view[1], token_seq=view[2], seq_starts=view[3], seq_lens=view[4],
        first_positions=view[5], state_slots=view[6], want_rows=view[7], block_tables=tables, request_ids=request_ids,
        host_q_lens=[1] * count, host_first_positions=[0] * count, host_state_slots=[0] * count, max_q_len=1,
        max_seq_len=max_positions, wants_every_row_in_order=True,
    )
    return ctx, offsets


def decode_layout(count: int, table_width: int, groups: int) -> list[int]:
    """Section sizes (int32 words) of a decode step's buffer."""
    return [count, count, count, count + 1, count, count, count, count] + [count * table_width] * groups
