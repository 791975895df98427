"""Trace scripts: the same requests cut into steps in different ways.

A trace is a list of steps {"step", "entries": [{"id", "tokens", "want"}], "end": [...]}, the
format `bin/trace_run` reads. Every entry asks for the logits of all its tokens, so each way
of cutting yields logits for every (request, position) and all can be compared with the
plain implementation's whole-sequence logits.
"""
from __future__ import annotations

import math


def whole(requests: dict) -> list:
    """Each request alone and whole: one step per request."""
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def prompt_then_decode(requests: dict, tail: int = 32) -> list:
    """Most of it in one step, the last `tail` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head],
                                                        "want": list(range(head))}], "end": []})
        for p in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[p:p + 1], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def all_together(requests: dict, tail: int = 4) -> list:
    """Every request's head in one step, then their last `tail` tokens one step each, all requests side by side:
    decode steps with as many rows as there are requests."""
    heads = {rid: max(1, len(toks) - tail) for rid, toks in requests.items()}
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": toks[:heads[rid]], "want": list(range(heads[rid]))}
                                     for rid, toks in requests.items()], "end": []}]
    longest = max(len(toks) - heads[rid] for rid, toks in requests.items())
    for k in range(longest):
        entries, end = [], []
        for rid, toks in requests.items():
            p = heads[rid] + k
            if p < len(toks):
                entries.append({"id": rid, "tokens": toks[p:p + 1], "want": [0]})
                if p == len(toks) - 1:
                    end.append(rid)
        steps.append({"step": len(steps), "entries": entries, "end": end})
    for rid, toks in requests.items():        # a request that is all head ends with the first step
        if heads[rid] == len(toks):
            steps[0]["end"].append(rid)
    return steps


def changing_portions(requests: dict, sizes=(7, 2, 33, 3, 16, 2, 64, 5)) -> list:
    """Each request alone, in portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in requests.items():
        lo, k = 0, 0
        while lo < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - lo)
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[lo:lo + n],
                                                            "want": list(range(n))}],
                          "end": [rid] if lo + n == len(toks) else []})
            lo += n
            k += 1
    return steps


def mixed(requests: dict, max_live: int = 4, portion: int = 24, prefill_share: float = 0.6) -> list:
    """Up to `max_live` requests at a time: each is fed in portions until `prefill_share` of it is in,
    then one token per step (as if decoded), while the others' portions ride in the same batch. A
    request that ends frees its pages, and the next one waiting takes them."""
    waiting = list(requests.items())
    live = {}   # rid -> [tokens, fed, prefill_end]
    steps = []
    turn = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0, max(1, min(len(toks), math.ceil(len(toks) * prefill_share)))]
        entries, ended = [], []
        for j, (rid, st) in enumerate(list(live.items())):
            toks, fed, pre = st
            if fed < pre:
                if (turn + j) % 3 == 2 and len(live) > 1:
                    continue  # this request sits a step out and goes on later
                n = min(portion - 5 * (j % 3), pre - fed)
                n = max(2, n) if pre - fed >= 2 else pre - fed
            else:
                n = 1
            entries.append({"id": rid, "tokens": toks[fed:fed + n], "want": list(range(n))})
            st[1] = fed + n
            if st[1] == len(toks):
                ended.append(rid)
        for rid in ended:
            del live[rid]
        steps.append({"step": len(steps), "entries": entries, "end": ended})
        turn += 1
    return steps


def peak_tokens(steps: list, round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each request's count rounded up to `round_to`."""
    held, peak = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def collect(steps: list, logits_of_step) -> dict:
    """{(request, position): logits row} from a replay; `logits_of_step(step)` gives [wanted, vocab] or None."""
    out, fed = {}, {}
    for st in steps:
        rows = logits_of_step(st)
        r = 0
        for e in st["entries"]:
            base = fed.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], base + w)] = rows[r]
                r += 1
            fed[e["id"]] = base + len(e["tokens"])
        for rid in st["end"]:
            fed.pop(rid, None)
    return out


def scheduled(requests: dict, prompt_lens: dict, max_live: int = 4, portions=(300, 129, 512, 200, 257, 140)) -> list:
    """Steps of the form the scheduler makes: ONE portion of a prompt first (the head of the line of prompts, which
    then goes to the back of it), then one row for every request that is decoding, in order of admission. The
    first `prompt_lens[rid]` tokens of a request are its prompt, the rest is fed one token a step as if it had
    been decoded. Requests are admitted in order while fewer than `max_live` are live. The portion sizes cycle
    through `portions`, so portions of more than one and more than two 128-row tiles stand beside single rows."""
    waiting = list(requests.items())
    live, line = {}, []        # rid -> [tokens, fed, prompt_len]; the line of prompts that still have portions to run
    steps, k = [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0, max(1, min(len(toks), prompt_lens[rid]))]
            line.append(rid)
        entries, ended = [], []
        if line:
            rid = line.pop(0)
            toks, fed, pre = live[rid]
            n = min(portions[k % len(portions)], pre - fed)
            k += 1
            entries.append({"id": rid, "tokens": toks[fed:fed + n], "want": list(range(n))})
            live[rid][1] = fed + n
            if fed + n < pre:
                line.append(rid)
            portion_of = rid
        else:
            portion_of = None
        for rid, st in live.items():
            toks, fed, pre = st
            if rid == portion_of or rid in line or fed < pre or fed >= len(toks):
                continue
            entries.append({"id": rid, "tokens": toks[fed:fed + 1], "want": [0]})
            st[1] = fed + 1
        for rid, st in list(live.items()):
            if st[1] == len(st[0]):
                ended.append(rid)
                del live[rid]
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def shape_of(steps: list) -> list:
    """For every step (rows of its leading multi-row entries, single-row entries behind them), or None where a
    multi-row entry follows a single row: the scheduler never forms such a step."""
    out = []
    for st in steps:
        sizes = [len(e["tokens"]) for e in st["entries"]]
        multi = [n for n in sizes if n > 1]
        ok = sizes[:len(multi)] == multi
        out.append((sum(multi), len(sizes) - len(multi)) if ok else None)
    return out
