"""Builders of replay traces: the same requests cut in different ways.

Every builder returns ``(steps, places, max_tokens)``: the JSON steps for ``bin/trace_run``,
for each step the ``(request, position)`` of every wanted row in file order, and the most tokens
live requests hold at any time (each request's count rounded up to 64), which sizes the pool.
"""

from __future__ import annotations

import random
from typing import Dict, List, Sequence, Tuple

from helpers import round_up

Steps = List[dict]
Places = Dict[int, List[Tuple[str, int]]]


class _Builder:
    def __init__(self, thin: int = 0):
        # thin > 0: of the places a builder wants, keep a portion's first and last and every
        # position that is a multiple of ``thin`` (wide vocabularies make every row expensive)
        self.thin = int(thin)
        self.steps: Steps = []
        self.places: Places = {}
        self.fed: Dict[str, int] = {}
        self.peak = 0

    def step(self, feeds: Sequence[Tuple[str, List[int], List[int]]], end: Sequence[str] = ()):
        """feeds: (request, tokens, want indices into tokens)."""
        n = len(self.steps)
        entries, places = [], []
        for rid, toks, want in feeds:
            start = self.fed.get(rid, 0)
            if self.thin:
                want = [w for w in want if w in (0, len(toks) - 1) or (start + w) % self.thin == 0]
            entries.append({"id": rid, "tokens": list(toks), "want": list(want)})
            places += [(rid, start + w) for w in want]
            self.fed[rid] = start + len(toks)
        self.peak = max(self.peak, sum(round_up(v, 64) for v in self.fed.values()))
        self.steps.append({"step": n, "entries": entries, "end": list(end)})
        if places:
            self.places[n] = places
        for rid in end:
            del self.fed[rid]

    def result(self):
        return self.steps, self.places, self.peak


def whole(reqs: Dict[str, List[int]], thin: int = 0):
    """Each request alone and whole, one step each, every position wanted."""
    b = _Builder(thin)
    for rid, toks in reqs.items():
        b.step([(rid, toks, list(range(len(toks))))], end=[rid])
    return b.result()


def tail_one_by_one(reqs: Dict[str, List[int]], tail: int = 32, thin: int = 0):
    """Most of each request in one step, the last ``tail`` tokens one by one."""
    b = _Builder(thin)
    for rid, toks in reqs.items():
        head = max(len(toks) - tail, 0)
        if head:
            b.step([(rid, toks[:head], list(range(head)))])
        for i in range(head, len(toks)):
            b.step([(rid, [toks[i]], [0])], end=[rid] if i == len(toks) - 1 else [])
    return b.result()


def portions(reqs: Dict[str, List[int]], sizes=(2, 3, 5, 24, 7, 2, 16, 9, 2, 31, 4), thin: int = 0):
    """Each request in portions of changing size, down to two tokens."""
    b = _Builder(thin)
    k = 0
    for rid, toks in reqs.items():
        i = 0
        while i < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - i)
            k += 1
            last = i + n == len(toks)
            b.step([(rid, toks[i:i + n], list(range(n)))], end=[rid] if last else [])
            i += n
    return b.result()


def mixed(reqs: Dict[str, List[int]], seed: int = 0, live_max: int = 4, tail: int = 12,
          chunks=(2, 3, 5, 8, 13, 24, 40), thin: int = 0):
    """Up to ``live_max`` live requests: portions of some beside single decoded tokens of others,
    requests now and then left out of a step; finished requests end, new ones take their pages."""
    rng = random.Random(seed)
    b = _Builder(thin)
    waiting = list(reqs.items())
    live: List[Tuple[str, List[int]]] = []
    while waiting or live:
        while waiting and len(live) < live_max:
            live.append(waiting.pop(0))
        feeds, ending = [], []
        for rid, toks in live:
            done = b.fed.get(rid, 0)
            if len(live) > 1 and rng.random() < 0.2:
                continue                                   # left out of this step
            left = len(toks) - done
            if left > tail:
                n = min(left - tail, rng.choice(list(chunks)))
            else:
                n = 1
            want = list(range(n)) if n <= 8 else sorted({0, n // 2, n - 2, n - 1})
            feeds.append((rid, toks[done:done + n], want))
            if done + n == len(toks):
                ending.append(rid)
        if not feeds:
            continue
        b.step(feeds, end=ending)
        live = [(rid, toks) for rid, toks in live if rid not in ending]
    return b.result()
