"""Builders of replay traces (the JSON steps `bin/trace_run` reads) for the ways of cutting work
that the tests compare, and a runner that collects logits by (request, position)."""
from __future__ import annotations

import itertools

import numpy as np


def prompt(seed: int, n: int, vocab: int) -> list[int]:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def whole(reqs: dict[str, list[int]]) -> list[dict]:
    """Each request alone, its whole sequence in one step, every position wanted."""
    return [{"step": i, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))}], "end": [r]} for i, (r, t) in enumerate(reqs.items())]


def tail_one_by_one(reqs: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of a sequence in one step, then the last `tail` tokens one per step."""
    steps, n = [], 0
    for r, t in reqs.items():
        head = max(1, len(t) - tail)
        steps.append({"step": n, "entries": [{"id": r, "tokens": t[:head], "want": list(range(head))}], "end": []})
        n += 1
        for i in range(head, len(t)):
            steps.append({"step": n, "entries": [{"id": r, "tokens": [t[i]], "want": [0]}], "end": []})
            n += 1
        steps[-1]["end"] = [r]
    return steps


def portions(reqs: dict[str, list[int]], sizes=(7, 5, 3, 2)) -> list[dict]:
    """Each request alone, cut into portions of changing size, down to two tokens."""
    steps, n = [], 0
    for r, t in reqs.items():
        at = 0
        for size in itertools.cycle(sizes):
            if at >= len(t):
                break
            part = t[at:at + size]
            steps.append({"step": n, "entries": [{"id": r, "tokens": part, "want": list(range(len(part)))}], "end": []})
            at += len(part)
            n += 1
        steps[-1]["end"] = [r]
    return steps


def mixed(reqs: dict[str, list[int]], max_live: int = 4, seed: int = 0, decode_tail: int = 12, sizes=(2, 3, 5, 9, 17)) -> list[dict]:
    """Up to `max_live` requests at a time: portions of some beside single tokens of others, a
    request sometimes left out of a step, new requests admitted as old ones end."""
    rng = np.random.default_rng(seed)
    waiting = list(reqs.items())
    live: dict[str, int] = {}
    steps, n = [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            r, _ = waiting.pop(0)
            live[r] = 0
        entries, end = [], []
        for r in list(live):
            t, at = reqs[r], live[r]
            if len(live) > 1 and rng.random() < 0.2:
                continue  # left out of this step
            left = len(t) - at
            size = 1 if left <= decode_tail else int(min(left - decode_tail, rng.choice(list(sizes))))
            part = t[at:at + size]
            entries.append({"id": r, "tokens": part, "want": list(range(len(part)))})
            live[r] = at + len(part)
            if live[r] == len(t):
                end.append(r)
                del live[r]
        if not entries:
            continue
        steps.append({"step": n, "entries": entries, "end": end})
        n += 1
    return steps


def max_live_tokens(steps: list[dict], round_to: int = 64) -> int:
    """The --max-tokens a trace needs: the most tokens live requests hold at any time, each
    request's count rounded up to a multiple of `round_to`."""
    held: dict[str, int] = {}
    most = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        most = max(most, sum(-(-v // round_to) * round_to for v in held.values()))
        for r in s["end"]:
            held.pop(r, None)
    return most


def run_steps(runner, steps: list[dict]) -> dict[tuple[str, int], np.ndarray]:
    """Drive a ModelRunner through a trace in-process; logits rows by (request, position)."""
    from inference_bench_b200.engine.step import StepEntry

    out = {}
    at: dict[str, int] = {}
    for s in steps:
        entries = []
        for e in s["entries"]:
            if not runner.cache.has(e["id"]):
                runner.cache.admit(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        logits = runner.step(entries)
        rows = logits.cpu().numpy() if logits is not None else None
        k = 0
        for e in s["entries"]:
            base = at.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], base + w)] = rows[k]
                k += 1
            at[e["id"]] = base + len(e["tokens"])
        for r in s["end"]:
            runner.cache.release(r)
    return out
