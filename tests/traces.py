"""Ways of cutting the same requests into steps, shared by the replay tests.

A trace is a list of steps; a step is ``{"entries": [(rid, tokens, want)], "end": [rid]}``.
``want`` holds places among the step's tokens.  Every builder asks for the
logits of every token it feeds unless told otherwise, so the result can be
compared position by position with the plain model's ``[S, V]`` logits.
"""

from __future__ import annotations

import random
from typing import Dict, List, Sequence, Tuple


def whole(requests: Dict[str, List[int]]) -> List[dict]:
    """Each request alone and whole, one step each."""
    return [{"entries": [(rid, toks, list(range(len(toks))))], "end": [rid]} for rid, toks in requests.items()]


def tail_decoded(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of each request in one step, the last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"entries": [(rid, toks[:head], list(range(head)))], "end": []})
        for i in range(head, len(toks)):
            steps.append({"entries": [(rid, toks[i:i + 1], [0])], "end": []})
        steps[-1]["end"] = [rid]
    return steps


def decoded_together(requests: Dict[str, List[int]], tail) -> List[dict]:
    """Every prompt whole in a step of its own (logits at its last place), then decode steps of all live
    requests together, one token each; ``tail`` (a number, or one per request) is how many tokens of a
    request are decoded, so requests with short tails leave on the way and the batch shrinks."""
    tails = {rid: (tail[rid] if isinstance(tail, dict) else tail) for rid in requests}
    steps = []
    fed = {}
    for rid, toks in requests.items():
        n = max(1, len(toks) - tails[rid])
        steps.append({"entries": [(rid, toks[:n], [n - 1])], "end": []})
        fed[rid] = n
    while any(fed[rid] < len(requests[rid]) for rid in requests):
        live = [rid for rid in requests if fed[rid] < len(requests[rid])]
        entries = [(rid, [requests[rid][fed[rid]]], [0]) for rid in live]
        for rid in live:
            fed[rid] += 1
        steps.append({"entries": entries, "end": [rid for rid in live if fed[rid] == len(requests[rid])]})
    return steps


def portions(requests: Dict[str, List[int]], sizes: Sequence[int] = (7, 2, 13, 3, 2, 5, 17, 2, 31, 4)) -> List[dict]:
    """Each request alone, in portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in requests.items():
        i, k = 0, 0
        while i < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - i)
            steps.append({"entries": [(rid, toks[i:i + n], list(range(n)))], "end": []})
            i += n
            k += 1
        steps[-1]["end"] = [rid]
    return steps


def mixed(requests: Dict[str, List[int]], max_live: int = 4, seed: int = 0, decode_tail: int = 12,
          max_portion: int = 11) -> List[dict]:
    """Up to ``max_live`` live requests: portions of some beside single decoded tokens of others;
    requests start when a place frees and end mid-trace; now and then a live request sits a step out."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: List[dict] = []
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live.append({"rid": rid, "toks": toks, "fed": 0, "prefill_end": max(1, len(toks) - decode_tail)})
        entries, end = [], []
        for r in live:
            if len(live) > 1 and rng.random() < 0.15:
                continue                                  # left out of this step, goes on later
            left_prefill = r["prefill_end"] - r["fed"]
            if left_prefill > 0:
                n = min(left_prefill, rng.randint(2, max_portion))
                if left_prefill - n == 1:                 # never leave a portion of one prompt token
                    n += 1
            else:
                n = 1
            toks = r["toks"][r["fed"]:r["fed"] + n]
            entries.append((r["rid"], toks, list(range(len(toks)))))
            r["fed"] += len(toks)
            if r["fed"] >= len(r["toks"]):
                end.append(r["rid"])
        if not entries:
            continue
        steps.append({"entries": entries, "end": end})
        live = [r for r in live if r["rid"] not in end]
    return steps


def live_token_peak(steps: List[dict], unit: int = 64) -> int:
    """Most tokens live requests hold at any time, each request rounded up to ``unit``."""
    held: Dict[str, int] = {}
    peak = 0
    for st in steps:
        for rid, toks, _ in st["entries"]:
            held[rid] = held.get(rid, 0) + len(toks)
        peak = max(peak, sum(-(-n // unit) * unit for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak
