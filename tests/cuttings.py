"""Ways of cutting the same requests into steps.  A trace is a list of steps in the
replay program's format: ``{"step", "entries": [{"id", "tokens", "want"}], "end"}``.
Every entry wants the logits of all its tokens, so each (request, position) is
checked whichever way it was cut."""
from __future__ import annotations

import random


def _entry(rid, toks):
    return {"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}


def whole(requests: dict[str, list[int]]):
    """Each request alone and whole: one step per request."""
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [_entry(rid, toks)], "end": [rid]})
    return steps


def tail_decode(requests, tail=32):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [_entry(rid, toks[:head])], "end": []})
        for j in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [_entry(rid, toks[j:j + 1])], "end": []})
        steps[-1]["end"] = [rid]
    return steps


def portions(requests, sizes=(7, 2, 13, 5, 2, 3, 11, 2, 17)):
    """Portions of changing size, down to two tokens."""
    steps = []
    k = 0
    for rid, toks in requests.items():
        i = 0
        while i < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - i)
            k += 1
            steps.append({"step": len(steps), "entries": [_entry(rid, toks[i:i + n])], "end": []})
            i += n
        steps[-1]["end"] = [rid]
    return steps


def mixed(requests, max_live=4, seed=0, prefill_sizes=(9, 2, 16, 5, 23, 3), decode_tail=12):
    """Up to ``max_live`` requests at a time; in each step some feed a portion of their
    prompt, others a single token (their last ``decode_tail`` tokens go one by one), some
    sit the step out.  Requests start when a place frees up, so pages are used again.
    Returns (steps, peak tokens held at once with each request rounded up to 64)."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: dict[str, list] = {}     # rid -> [tokens, fed]
    steps = []
    peak = 0
    k = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0]
        entries, ended = [], []
        for rid in list(live):
            toks, fed = live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue                       # left out of this step
            left = len(toks) - fed
            if left > decode_tail:
                n = min(prefill_sizes[k % len(prefill_sizes)], left - decode_tail)
                k += 1
            else:
                n = 1
            entries.append(_entry(rid, toks[fed:fed + n]))
            live[rid][1] = fed + n
        held = sum(-(-max(v[1], 1) // 64) * 64 for v in live.values())
        peak = max(peak, held)
        for rid in list(live):
            if live[rid][1] == len(live[rid][0]):
                ended.append(rid)
                del live[rid]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ended})
        elif ended:
            steps[-1]["end"] += ended
    return steps, peak


def peak_tokens(steps):
    """Most tokens held at once over a trace, each request rounded up to a multiple of 64."""
    held: dict[str, int] = {}
    peak = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // 64) * 64 for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def run_trace(engine, steps):
    """Drives ``engine.step`` with a trace; returns {(request, position): logits row (cpu)}."""
    import torch
    slots, fed, out = {}, {}, {}
    for st in steps:
        items = []
        for e in st["entries"]:
            rid = e["id"]
            if rid not in slots:
                slots[rid] = engine.cache.open()
                assert slots[rid] >= 0
                fed[rid] = 0
            items.append((slots[rid], e["tokens"], e["want"]))
        logits = engine.step(items).to("cpu", torch.float32)
        engine.rt.ops.check_errors()
        row = 0
        for e in st["entries"]:
            for w in e["want"]:
                out[(e["id"], fed[e["id"]] + w)] = logits[row]
                row += 1
            fed[e["id"]] += len(e["tokens"])
        for rid in st["end"]:
            engine.cache.close(slots.pop(rid))
        assert engine.cache.manager.check() == ""
    return out
