"""Builders of replay traces: the same requests fed whole, with a decoded tail, in portions of changing size,
and mixed with other requests. A trace is a list of steps in the replay program's input format:

    {"step": i, "entries": [{"id": "a", "tokens": [...], "want": [...]}, ...], "end": ["a", ...]}

Every builder asks for the logits of every token it feeds, so each (request, position) can be compared with
the plain implementation's whole-sequence forward.
"""

from __future__ import annotations

import random


def whole(requests: dict[str, list[int]]) -> list[dict]:
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def decoded_tail(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of a request in one step, its last `tail` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for i in range(head, len(toks)):
            steps.append({"entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    return [{"step": i, **s} for i, s in enumerate(steps)]


def portions(requests: dict[str, list[int]], sizes=(7, 2, 13, 3, 2, 29, 2, 16, 5, 17, 2, 64, 3)) -> list[dict]:
    """Each request alone, in portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in requests.items():
        at, j = 0, 0
        while at < len(toks):
            n = min(sizes[j % len(sizes)], len(toks) - at)
            steps.append({"entries": [{"id": rid, "tokens": toks[at:at + n], "want": list(range(n))}], "end": []})
            at += n
            j += 1
        steps[-1]["end"] = [rid]
    return [{"step": i, **s} for i, s in enumerate(steps)]


def mixed(requests: dict[str, list[int]], live: int = 4, seed: int = 0, decode_after: float = 0.6) -> list[dict]:
    """Up to `live` requests at a time. Each step every live request brings either a portion of its text (2 to
    19 tokens) or, once past `decode_after` of its text, a single token, and sometimes sits a step out. A request
    that ends makes room for the next, so pages freed by one are taken by another."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    running: list[list] = []       # [id, tokens, fed]
    steps = []
    while waiting or running:
        while waiting and len(running) < live:
            rid, toks = waiting.pop(0)
            running.append([rid, toks, 0])
            if rng.random() < 0.5:
                break               # stagger the arrivals
        entries, end = [], []
        for r in running:
            rid, toks, fed = r
            if len(running) > 1 and rng.random() < 0.15:
                continue            # left out of this step, goes on later
            left = len(toks) - fed
            n = 1 if fed >= decode_after * len(toks) else min(left, rng.choice([2, 2, 3, 5, 8, 11, 16, 19]))
            entries.append({"id": rid, "tokens": toks[fed:fed + n], "want": list(range(n))})
            r[2] += n
            if r[2] == len(toks):
                end.append(rid)
        if not entries:
            continue
        running = [r for r in running if r[0] not in end]
        steps.append({"entries": entries, "end": end})
    return [{"step": i, **s} for i, s in enumerate(steps)]


def tokens_held(trace: list[dict], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each request's count rounded up to `round_to`."""
    held: dict[str, int] = {}
    most = 0
    for s in trace:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        most = max(most, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return most


def live_at_once(trace: list[dict]) -> int:
    live, most = set(), 0
    for s in trace:
        live |= {e["id"] for e in s["entries"]}
        most = max(most, len(live))
        live -= set(s["end"])
    return most
