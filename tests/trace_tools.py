"""Building traces (the JSON steps trace_run reads) that cut the same requests in different ways."""
from __future__ import annotations

import numpy as np
import torch


def make_requests(vocab: int, lengths: list[int], seed: int) -> dict[str, list[int]]:
    rng = np.random.default_rng(seed)
    return {f"r{i}": [int(t) for t in rng.integers(0, vocab, size=n)] for i, n in enumerate(lengths)}


def whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole: one step, every position wanted."""
    return [
        {"step": i, "entries": [{"id": rid, "tokens": tokens, "want": list(range(len(tokens)))}], "end": [rid]}
        for i, (rid, tokens) in enumerate(requests.items())
    ]


def tail_decode(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of a request in one step, then its last ``tail`` tokens one by one."""
    steps = []
    for rid, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": tokens[:head], "want": [head - 1]}], "end": []})
        for i in range(head, len(tokens)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [tokens[i]], "want": [0]}], "end": [rid] if i == len(tokens) - 1 else []})
        if head == len(tokens):
            steps[-1]["end"] = [rid]
    return steps


def portions(requests: dict[str, list[int]], sizes=(7, 5, 3, 2, 2, 11, 2, 4, 64, 2, 16, 3)) -> list[dict]:
    """Each request alone in portions of changing size, down to two tokens; the last place of each portion wanted."""
    steps = []
    for rid, tokens in requests.items():
        at, k = 0, 0
        while at < len(tokens):
            n = min(sizes[k % len(sizes)], len(tokens) - at)
            k += 1
            at += n
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": tokens[at - n : at], "want": [n - 1, 0] if n > 1 else [0]}],
                          "end": [rid] if at == len(tokens) else []})
    return steps


def mixed(requests: dict[str, list[int]], seed: int, max_live: int = 4, tail: int = 32, max_portion: int = 24, page_size: int = 64) -> tuple[list[dict], int]:
    """Up to ``max_live`` requests at once: portions of some beside single tokens of others, some left out of a step.

    Returns the steps and the largest number of tokens (each request rounded up to whole
    pages) live at any time: a pool of exactly that size forces pages to be used again.
    """
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    live: dict[str, int] = {}
    steps: list[dict] = []
    peak = 0
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.6):
            rid, _ = waiting.pop(0)
            live[rid] = 0
        entries, ended = [], []
        for rid in list(live):
            if len(live) > 1 and rng.random() < 0.25:
                continue  # left out of this step, goes on later
            tokens, at = requests[rid], live[rid]
            decode_from = max(1, len(tokens) - tail)
            if at >= decode_from:
                n = 1
            else:
                n = int(min(decode_from - at, rng.integers(2, max_portion + 1)))
                if decode_from - at - n == 1:
                    n += 1  # never leave a one-token remainder of the prompt part
            want = [n - 1] if rng.random() < 0.8 or n == 1 else []
            entries.append({"id": rid, "tokens": tokens[at : at + n], "want": want})
            live[rid] = at + n
        held = sum(-(-at // page_size) * page_size for at in live.values())
        peak = max(peak, held)
        for rid in list(live):
            if live[rid] == len(requests[rid]):
                ended.append(rid)
                del live[rid]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps, peak


def expected_rows(steps: list[dict], full_logits: dict[str, torch.Tensor]) -> dict[int, torch.Tensor]:
    """For every step that wants something: the plain implementation's logits at the wanted places."""
    at = {rid: 0 for rid in full_logits}
    out = {}
    for step in steps:
        rows = []
        for entry in step["entries"]:
            for w in entry.get("want", []):
                rows.append(full_logits[entry["id"]][at[entry["id"]] + w])
            at[entry["id"]] += len(entry["tokens"])
        if rows:
            out[step["step"]] = torch.stack(rows)
    return out


def run_and_compare(runner, steps: list[dict], full_logits: dict[str, torch.Tensor], atol: float, rtol: float = 0.0) -> float:
    """Replay the steps through the engine's step function; returns the largest error seen."""
    from tinyllama_inference_engine_b200.engine.replay import replay_step

    expected = expected_rows(steps, full_logits)
    worst = 0.0
    for step in steps:
        got = replay_step(runner, step)
        if step["step"] in expected:
            want = expected[step["step"]]
            assert got is not None and got.shape == want.shape, (step["step"], None if got is None else got.shape, want.shape)
            error = (got - want).abs()
            bound = atol + rtol * want.abs()
            if not bool((error <= bound).all()):
                row = int((error - bound).max(1).values.argmax())
                raise AssertionError(
                    f"step {step['step']}: wanted row {row} differs by {float(error[row].max()):.3e} (bound {atol:.1e}); entries "
                    + str([(e['id'], len(e['tokens']), e.get('want')) for e in step['entries']])
                )
            worst = max(worst, float(error.max()))
        else:
            assert got is None
    return worst
