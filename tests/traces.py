"""Builders of replay traces: the same requests cut into steps in different ways.

A trace is a list of step messages as ``bin/trace_run`` reads them.  Every builder asks for
the logits of every token it feeds, so that any two traces of the same requests can be
compared position by position.  ``collect`` runs a trace and files the logits by
(request, position).
"""

from __future__ import annotations

import random


def whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone, in one step."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def decode_tail(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for i in range(head, len(toks)):
            steps.append({"entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    for i, s in enumerate(steps):
        s["step"] = i
    return steps


def portions(requests: dict[str, list[int]], sizes=(7, 2, 5, 3, 16, 2, 11, 4)) -> list[dict]:
    """Each request in portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in requests.items():
        at, k = 0, 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            steps.append({"entries": [{"id": rid, "tokens": toks[at:at + n], "want": list(range(n))}], "end": []})
            at += n
            k += 1
        steps[-1]["end"] = [rid]
    for i, s in enumerate(steps):
        s["step"] = i
    return steps


def mixed(requests: dict[str, list[int]], max_live: int = 4, seed: int = 0, prompt_frac: float = 0.6,
          max_portion: int = 9, min_portion: int = 2, stagger: int = 0) -> list[dict]:
    """Up to ``max_live`` requests at a time: the first ``prompt_frac`` of each is fed in random
    portions (``min_portion`` to ``max_portion`` tokens, >= 2 where possible), the rest token by
    token, beside whatever the other live requests bring; some steps leave a request out.  Requests
    start as others end, so with a small pool their pages are the ones just given back.  With
    ``stagger`` a request starts no sooner than that many steps after the one before it, so that
    prompts of some run beside decoded tokens of others."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: dict[str, dict] = {}
    steps = []
    last_start = -stagger
    while waiting or live:
        while waiting and len(live) < max_live and (len(steps) - last_start >= stagger or not live):
            rid, toks = waiting.pop(0)
            last_start = len(steps)
            live[rid] = {"toks": toks, "at": 0, "prompt": max(1, int(len(toks) * prompt_frac))}
        entries, end = [], []
        for rid, st in list(live.items()):
            if len(live) > 1 and rng.random() < 0.2:
                continue                                    # left out of this step
            left_prompt = st["prompt"] - st["at"]
            if left_prompt > 0:
                n = min(left_prompt, rng.randint(min_portion, max_portion))
                if left_prompt - n == 1:
                    n += 1
            else:
                n = 1
            toks = st["toks"][st["at"]:st["at"] + n]
            entries.append({"id": rid, "tokens": toks, "want": list(range(len(toks)))})
            st["at"] += len(toks)
            if st["at"] >= len(st["toks"]):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def max_live_tokens(steps: list[dict], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: dict[str, int] = {}
    peak = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


def collect(run_step, steps: list[dict]) -> dict[tuple[str, int], "object"]:
    """Runs ``steps`` through ``run_step(msg) -> array [wanted, vocab] | None`` and returns
    {(request, position): logits row}."""
    fed: dict[str, int] = {}
    out = {}
    for s in steps:
        res = run_step(s)
        row = 0
        for e in s["entries"]:
            base = fed.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], base + w)] = res[row]
                row += 1
            fed[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            fed.pop(rid, None)
        assert res is None or row == len(res)
    return out
