"""The filters a sampled request runs with when it names none (the reference's `server/sampling_defaults.py:41-66`).

A request that sends a temperature alone would sample the whole vocabulary (top_p 1, top_k 0), which is not what a
checkpoint was tuned for: its card (generation_config.json) recommends a top_k and a top_p. The first of these that says
anything decides all three filters:

  1. the request: any of top_p / top_k / min_p given, the fields it leaves out taking the caller's flags below;
  2. the flags the program was started with;
  3. the card: its top_p and top_k, min_p 0;
  4. none: top_p 1, top_k 0, min_p 0.

Only the filters move: the temperature stays the request's, a greedy request is untouched. A sampled request that names
no seed draws its own (63 bits from the operating system: `SamplingParams.resolved_seed`), so that its answer can be had
again from the seed on record.
"""

from __future__ import annotations

import json
import os

FIELDS = ("top_p", "top_k", "min_p")
PLAIN = {"top_p": 1.0, "top_k": 0, "min_p": 0.0}


def _number(key: str, value):
    return int(value) if key == "top_k" else float(value)


def resolve(request: dict | None, flags: dict | None = None, card: dict | None = None) -> dict:
    """{top_p, top_k, min_p, source} for one request; `source` is "request", "flags", "card" or "none". Fields that
    are absent or None were not given."""
    flags = {k: v for k, v in (flags or {}).items() if k in FIELDS and v is not None}
    sent = {k: v for k, v in (request or {}).items() if k in FIELDS and v is not None}
    if sent:
        base = dict(PLAIN, **flags)
        return dict({k: _number(k, sent.get(k, base[k])) for k in FIELDS}, source="request")
    if flags:
        return dict({k: _number(k, flags.get(k, PLAIN[k])) for k in FIELDS}, source="flags")
    if card:
        return {"top_p": float(card.get("top_p", 1.0)), "top_k": int(card.get("top_k", 0) or 0), "min_p": 0.0, "source": "card"}
    return dict(PLAIN, source="none")


def card_sampling(folder: str) -> dict | None:
    """What a model folder's generation_config.json recommends for sampling ({top_p, top_k} where it names them), or
    None."""
    path = os.path.join(folder, "generation_config.json")
    if not os.path.isfile(path):
        return None
    with open(path) as f:
        raw = json.load(f)
    card = {k: raw[k] for k in ("top_p", "top_k") if raw.get(k) is not None}
    return card or None
