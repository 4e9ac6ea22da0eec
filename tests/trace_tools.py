"""Builders of replay traces: whole, tail decoded one by one, changing portions, mixed."""

from __future__ import annotations

import random
from typing import Callable, Iterable

Wanted = Callable[[int], bool] | None      # which positions of a sequence are asked for; None = all


def _want(start: int, size: int, wanted: Wanted) -> list[int]:
    return [place for place in range(size) if wanted is None or wanted(start + place)]


def whole(request_id: str, tokens: list[int], step: int = 0, wanted: Wanted = None) -> list[dict]:
    return [{"step": step, "entries": [{"id": request_id, "tokens": tokens, "want": _want(0, len(tokens), wanted)}],
             "end": [request_id]}]


def tail_one_by_one(request_id: str, tokens: list[int], tail: int = 32, step: int = 0, wanted: Wanted = None) -> list[dict]:
    """Most of the sequence in one step, the last ``tail`` tokens one by one."""
    tail = min(tail, len(tokens) - 1)
    head = tokens[: len(tokens) - tail]
    records = [{"step": step, "entries": [{"id": request_id, "tokens": head, "want": _want(0, len(head), wanted)}], "end": []}]
    for offset, token in enumerate(tokens[len(head):]):
        records.append({"step": step + 1 + offset, "entries": [{"id": request_id, "tokens": [token], "want": [0]}], "end": []})
    records[-1]["end"] = [request_id]
    return records


def portions(request_id: str, tokens: list[int], sizes: Iterable[int], step: int = 0, wanted: Wanted = None) -> list[dict]:
    """The sequence in portions of the given sizes (cycled)."""
    records, at, sizes = [], 0, list(sizes)
    index = 0
    while at < len(tokens):
        size = min(sizes[index % len(sizes)], len(tokens) - at)
        chunk = tokens[at : at + size]
        records.append({"step": step + index, "entries": [{"id": request_id, "tokens": chunk, "want": _want(at, size, wanted)}], "end": []})
        at += size
        index += 1
    records[-1]["end"] = [request_id]
    return records


def mixed(sequences: dict[str, list[int]], seed: int, max_live: int = 4, page: int = 16,
          prompt_fraction: float = 0.6, wanted: Wanted = None) -> tuple[list[dict], int]:
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of others.

    Each request feeds the first ``prompt_fraction`` of its tokens in portions of random size
    (2 and up) and the rest one token a step; a request sometimes sits a step out; when one
    ends the next in line starts.  Returns the records and the peak number of tokens live
    requests held, each rounded up to whole pages (for sizing the pool so pages are reused).
    """
    rng = random.Random(seed)
    waiting = list(sequences)
    live: dict[str, int] = {}          # id -> tokens fed so far
    records, peak, step = [], 0, 0
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.7):
            live[waiting.pop(0)] = 0
        entries, ended = [], []
        for request_id in list(live):
            tokens, fed = sequences[request_id], live[request_id]
            if fed > 0 and len(live) > 1 and rng.random() < 0.15:
                continue  # sits this step out
            prompt_len = max(2, int(len(tokens) * prompt_fraction))
            if fed < prompt_len:
                size = min(rng.choice([2, 3, 5, 7, 13, 16, 17, 31, 33]), prompt_len - fed)
                if prompt_len - fed - size == 1:
                    size += 1  # never leave a one-token prompt tail
            else:
                size = 1
            size = min(size, len(tokens) - fed)
            chunk = tokens[fed : fed + size]
            entries.append({"id": request_id, "tokens": chunk, "want": _want(fed, size, wanted)})
            live[request_id] = fed + size
            if live[request_id] == len(tokens):
                ended.append(request_id)
        held = sum(-(-count // page) * page for count in live.values())
        peak = max(peak, held)
        if entries:
            rng.shuffle(entries)
            records.append({"step": step, "entries": entries, "end": ended})
            step += 1
        for request_id in ended:
            del live[request_id]
    return records, peak


def collect(records: list[dict], outputs: dict[int, "object"]) -> dict[str, dict[int, "object"]]:
    """``request -> position -> logits row`` from per-step outputs (arrays [wanted, vocab])."""
    fed: dict[str, int] = {}
    rows: dict[str, dict[int, object]] = {}
    for record in records:
        out = outputs.get(record["step"])
        at = 0
        for entry in record["entries"]:
            start = fed.get(entry["id"], 0)
            for place in entry.get("want", []):
                rows.setdefault(entry["id"], {})[start + place] = out[at]
                at += 1
            fed[entry["id"]] = start + len(entry["tokens"])
    return rows
