"""One step's batch: requests' next tokens, flattened, with everything a kernel needs to find the cache."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


ATTENTION_TILE_ROWS = 64   # rows of one work item of the prompt-attention kernel (csrc/attention_prefill.cu: PREFILL_ROWS)
ATTENTION_TC_TILE_ROWS = 128   # rows of one work item of the tensor-memory kernel (csrc/attention_prefill_tc.cu)


def paired_attention_tiles(q_lens: list[int], first_positions: list[int], seq_starts: list[int]) -> list[int]:
    """Work items of the tensor-memory attention kernel: (entry, first row, entry or -1, first row) per item.

    A run of ATTENTION_TC_TILE_ROWS rows late in a long request sees many keys, an early one few.  Pairing the heaviest
    tile with the lightest, the second heaviest with the second lightest, and so on, gives every CTA about the same
    number of key tiles, so the grid finishes together instead of waiting for the last heavy tiles.
    """
    singles = []
    for index, count in enumerate(q_lens):
        for offset in range(0, count, ATTENTION_TC_TILE_ROWS):
            rows = min(ATTENTION_TC_TILE_ROWS, count - offset)
            work = -(-(first_positions[index] + offset + rows) // 64)
            singles.append((work, index, seq_starts[index] + offset))
    singles.sort(key=lambda item: -item[0])
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
      attn_tiles[N, 2]            (entry, first row) of every run of up to ATTENTION_TILE_ROWS consecutive rows of one entry:
                                  the work list of the prompt-attention kernel
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
    attn_tiles: torch.Tensor | None = None
    wants_every_row_in_order: bool = False      # want_rows is 0, 1, ..., num_tokens - 1
    attn_tiles_tc: torch.Tensor | None = None   # work items of the tensor-memory kernel: pairs of 128-row runs (int32 [n, 4])

    @property
    def decode_only(self) -> bool:
        return self.max_q_len == 1


def pack_step(entries: list[StepEntry], first_positions: list[int], slots: list[int], table_rows: list[list[list[int]]],
              device: torch.device) -> StepContext:
    """Flatten the entries into one int32 buffer, copy it once, and slice the views."""
    q_lens = [len(e.tokens) for e in entries]
    num_tokens, num_seqs = sum(q_lens), len(entries)
    token_ids: list[int] = []
    positions: list[int] = []
    token_seq: list[int] = []
    seq_starts = [0]
    want_rows: list[int] = []
    for index, (entry, first) in enumerate(zip(entries, first_positions)):
        start = seq_starts[-1]
        token_ids += entry.tokens
        positions += range(first, first + len(entry.tokens))
        token_seq += [index] * len(entry.tokens)
        want_rows += [start + w for w in entry.want]
        seq_starts.append(start + len(entry.tokens))
    seq_lens = [f + n for f, n in zip(first_positions, q_lens)]
    tiles: list[int] = []
    for index, count in enumerate(q_lens):
        for offset in range(0, count, ATTENTION_TILE_ROWS):
            tiles += [index, seq_starts[index] + offset]
    tiles_tc = paired_attention_tiles(q_lens, first_positions, seq_starts)
    sections = [token_ids, positions, token_seq, seq_starts, seq_lens, first_positions, slots, want_rows, tiles, tiles_tc]
    flat: list[int] = []
    offsets = []
    for section in sections:
        offsets.append((len(flat), len(section)))
        flat += section
    table_offsets = []
    for rows in table_rows:
        width = len(rows[0]) if rows else 0
        table_offsets.append((len(flat), num_seqs, width))
        for row in rows:
            flat += row
    host = torch.tensor(flat, dtype=torch.int32)
    if device.type == "cuda":
        host = host.pin_memory()
    buffer = host.to(device, non_blocking=True)
    views = [buffer[o : o + n] for o, n in offsets]
    tables = [buffer[o : o + b * w].view(b, w) for o, b, w in table_offsets]
    return StepContext(
        num_tokens=num_tokens, num_seqs=num_seqs,
        token_ids=views[0], positions=views[1], token_seq=views[2], seq_starts=views[3], seq_lens=views[4],
        first_positions=views[5], state_slots=views[6], want_rows=views[7] if want_rows else None,
        block_tables=tables, request_ids=[e.request_id for e in entries], host_q_lens=q_lens,
        host_first_positions=list(first_positions), host_state_slots=list(slots),
        max_q_len=max(q_lens), max_seq_len=max(seq_lens), attn_tiles=views[8].view(-1, 2),
        attn_tiles_tc=views[9].view(-1, 4), wants_every_row_in_order=want_rows == list(range(num_tokens)),
    )
