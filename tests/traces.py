"""Builders of replay traces: the same requests cut into steps in different ways."""
from __future__ import annotations


def whole(prompts: dict) -> list[dict]:
    """Each request alone, whole, every logit wanted."""
    steps = []
    for i, (rid, toks) in enumerate(prompts.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def tail_decoded(prompts: dict, tail: int = 32) -> list[dict]:
    """Most of a request in one step, its last `tail` tokens one by one."""
    steps, n = [], 0
    for rid, toks in prompts.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        n += 1
        for i in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
            n += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def portions(prompts: dict, sizes=(7, 2, 13, 3, 2, 29, 5, 2, 64, 2, 11)) -> list[dict]:
    """Portions of changing size, down to two tokens."""
    steps, n, k = [], 0, 0
    for rid, toks in prompts.items():
        at = 0
        while at < len(toks):
            m = min(sizes[k % len(sizes)], len(toks) - at)
            k += 1
            last = at + m == len(toks)
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[at:at + m], "want": list(range(m))}],
                          "end": [rid] if last else []})
            n += 1
            at += m
    return steps


def mixed(prompts: dict, max_live: int = 4, chunk=(9, 4, 17, 2, 6), decode_after: float = 0.6) -> list[dict]:
    """Up to `max_live` live requests: portions of some beside single tokens of others.
    A request is fed in portions up to `decode_after` of its length and token by token
    after that; a request starts as soon as one ends."""
    waiting = list(prompts.items())
    live: list[list] = []          # [rid, toks, at]
    steps, n, k = [], 0, 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live.append([rid, toks, 0])
        entries, end = [], []
        for slot, item in enumerate(live):
            rid, toks, at = item
            if (n + slot) % 5 == 4 and len(live) > 1:
                continue                                   # left out of this step, goes on later
            if at >= int(len(toks) * decode_after):
                m = 1
            else:
                m = min(chunk[k % len(chunk)], len(toks) - at)
                k += 1
            entries.append({"id": rid, "tokens": toks[at:at + m], "want": list(range(m))})
            item[2] = at + m
            if item[2] == len(toks):
                end.append(rid)
        live = [it for it in live if it[2] < len(it[1])]
        if entries:
            steps.append({"step": n, "entries": entries, "end": end})
            n += 1
    return steps


def collect(steps, outputs) -> dict:
    """(request id -> {position: logits row}) from the per-step arrays."""
    at = {}
    rows: dict = {}
    for st, out in zip(steps, outputs):
        r = 0
        for e in st["entries"]:
            base = at.get(e["id"], 0)
            for w in e["want"]:
                rows.setdefault(e["id"], {})[base + w] = out[r]
                r += 1
            at[e["id"]] = base + len(e["tokens"])
        assert out is None and r == 0 or r == len(out)
    return rows
