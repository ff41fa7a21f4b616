"""Continuous batching above the step function.

Reference: the driver ``LLM._generate_multiple`` (torchllms/inference/llm.py:761-997) runs
*static* batches: whole prompts in one forward (:999-1072), then one token per live request per
forward until each hits a stop id or its budget (:946-981); a batch larger than ``max_bsz`` is an
error (:883-886) and running out of pages raises (torchllms/models/paged_kv.py:285-289).  Kept
from it: the budget ``min(max_len - prompt_len, max_new_tokens)`` (:824-829), stop-on-any-of with
the stop token kept in the output and reported as ``stop_reason`` (:929-938, :972-981), an empty
result for a zero budget (:831-837), the last sampled token never being fed back (:905-908).

Here requests wait in arrival order, are admitted while a slot and pages are free, have their
prompts cut into portions under a per-step token budget, decode beside other requests' portions,
and leave as soon as they finish.  When pages run out: prompt portions are simply not scheduled
(or shortened); if even the decode tokens cannot get their pages, the running request admitted
last is pre-empted: its pages are freed and it goes back to the head of the queue to be
recomputed from its prompt and what it generated so far (its samples do not change, because
the sampling noise is keyed by request and token index).  A request that can never fit is
finished with an error instead of blocking the queue.
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Iterable, List, Optional, Sequence, Set, Tuple

from ..cache.manager import OutOfPages
from ..sampling.sampler import Sampler, SamplingParams
from .step import Engine, StepEntry


@dataclass
class Request:
    index: int                       # place in the caller's list: result order and sampling key
    prompt: List[int]
    budget: int                      # how many tokens it may generate
    sampling: SamplingParams = field(default_factory=SamplingParams)
    generated: List[int] = field(default_factory=list)
    stop_reason: Optional[int] = None
    error: Optional[str] = None
    finished: bool = False
    handle: Optional[int] = None
    n_fed: int = 0                   # tokens of prompt + generated that are in the cache
    n_preempted: int = 0

    def tokens(self) -> List[int]:
        return self.prompt + self.generated

    def span(self, start: int, n: int) -> List[int]:
        """Tokens ``start .. start + n`` of prompt followed by generated, without joining the two."""
        lp = len(self.prompt)
        if start + n <= lp:
            return self.prompt[start:start + n]
        if start >= lp:
            return self.generated[start - lp:start - lp + n]
        return self.prompt[start:] + self.generated[:start + n - lp]

    def n_pending(self) -> int:
        return len(self.prompt) + len(self.generated) - self.n_fed


@dataclass
class SchedulerStats:
    steps: int = 0
    tokens: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    max_running: int = 0
    decode_steps: int = 0            # steps that held decode tokens only
    decode_step_tokens: int = 0
    decode_seconds: float = 0.0      # wall time of those steps, sampling and its read-back included


class Scheduler:
    def __init__(self, engine: Engine, sampler: Sampler, *, max_num_seqs: Optional[int] = None,
                 max_num_batched_tokens: int = 2048, prefill_chunk: Optional[int] = None,
                 eos_ids: Iterable[int] = ()):
        self.engine = engine
        self.sampler = sampler
        self.max_num_seqs = min(int(max_num_seqs or engine.cache.max_num_seqs), engine.cache.max_num_seqs)
        self.max_num_batched_tokens = min(int(max_num_batched_tokens), engine.max_step_tokens)
        self.prefill_chunk = int(prefill_chunk or self.max_num_batched_tokens)
        if self.max_num_batched_tokens < 1 or self.prefill_chunk < 1:
            raise ValueError("token budget and prefill chunk must be at least 1")
        self.eos_set: Set[int] = set(int(t) for t in eos_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []      # in order of admission
        self.stats = SchedulerStats()
        self.trace: List[List[Tuple[int, int]]] = []   # per step: (request index, tokens fed)

    # ------------------------------------------------------------------ intake
    def add(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError(f"request {request.index}: empty prompt")
        if request.budget <= 0:
            request.finished = True          # nothing to generate: an empty result at once
            return
        page = self.engine.cache.page_size
        need = len(request.prompt) + request.budget - 1   # the last sampled token is never fed
        pool = min(g.allocator.n_pages for g in self.engine.cache.groups) * page if self.engine.cache.groups else need
        if need > self.engine.max_len or -(-need // page) * page > pool:
            request.finished = True
            request.error = (f"request needs {need} cached tokens but the engine holds at most "
                             f"{min(self.engine.max_len, pool)} for one request")
            return
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # --------------------------------------------------------------- one step
    def _room(self, planned: List[Tuple[Request, int]], req: Request, n: int) -> int:
        """Largest m <= n such that req may bring m tokens beside what is planned."""
        return min(n, self.engine.cache.room_for(req.handle, [(r.handle, k) for r, k in planned]))

    def _preempt(self, req: Request) -> None:
        self.engine.release(req.handle)
        req.handle = None
        req.n_fed = 0
        req.n_preempted += 1
        self.running.remove(req)
        self.waiting.appendleft(req)
        self.stats.preemptions += 1

    def _fail(self, req: Request, why: str) -> None:
        req.finished, req.error = True, why
        if req.handle is not None:
            self.engine.release(req.handle)
            req.handle = None
        if req in self.running:
            self.running.remove(req)

    def plan(self) -> List[Tuple[Request, int]]:
        """Decide which requests bring how many tokens to the next step.

        Decoding requests come first, one token each; then portions of prompts that are already
        running, oldest first; then new requests in arrival order.  If the decode tokens cannot
        get their pages, or nobody can move at all, the request admitted last is pre-empted and
        the plan is made again."""
        while True:
            decodes = [(r, 1) for r in self.running if r.n_pending() == 1 and r.n_fed > 0]
            if not self.engine.can_run([(r.handle, 1) for r, _ in decodes]):
                if len(self.running) == 1:
                    self._fail(self.running[0], "out of cache pages with nothing left to pre-empt")
                    return []
                self._preempt(self.running[-1])
                continue
            planned: List[Tuple[Request, int]] = decodes[: self.max_num_batched_tokens]
            budget = self.max_num_batched_tokens - len(planned)
            in_plan = {id(r) for r, _ in planned}
            for r in self.running:                         # portions of prompts already running
                if budget <= 0:
                    break
                if id(r) in in_plan:
                    continue
                n = self._room(planned, r, min(r.n_pending(), self.prefill_chunk, budget))
                if n > 0:
                    planned.append((r, n))
                    budget -= n
            while (self.waiting and budget > 0 and len(self.running) < self.max_num_seqs
                   and self.engine.cache.has_free_slot()):  # admission, in arrival order
                r = self.waiting[0]
                r.handle = self.engine.claim()
                want = min(r.n_pending(), self.prefill_chunk, budget)
                n = self._room(planned, r, want)
                # a newcomer must fit its first portion whole, unless it has the engine to itself
                if n < want and (self.running or n == 0):
                    self.engine.release(r.handle)
                    r.handle = None
                    break
                self.waiting.popleft()
                self.running.append(r)
                planned.append((r, n))
                budget -= n
            if planned or not self.running:
                break
            # requests are running but none can move: their prompts have eaten the pool
            if len(self.running) == 1:
                self._fail(self.running[0], "out of cache pages with nothing left to pre-empt")
                return []
            self._preempt(self.running[-1])
        self.stats.max_running = max(self.stats.max_running, len(self.running))
        return planned

    def step(self) -> List[Request]:
        """Plan, run and sample one step; returns the requests that finished in it."""
        before = [r for r in self.running]
        planned = self.plan()
        finished_now = [r for r in before if r.finished and r not in self.running]
        if not planned:
            if not finished_now and self.has_work() and not self.running:
                # nothing running and the head of the queue cannot start: it can never fit
                r = self.waiting.popleft()
                r.finished, r.error = True, "request does not fit the cache pool"
                finished_now.append(r)
            return finished_now
        entries, samplers = [], []
        for r, n in planned:
            toks = r.span(r.n_fed, n)
            completes = r.n_fed + n == len(r.prompt) + len(r.generated)
            entries.append(StepEntry(r.handle, toks, [n - 1] if completes else []))
            if completes:
                samplers.append(r)
        pure_decode = all(n == 1 and r.n_fed > 0 and r.generated for r, n in planned)
        t0 = time.perf_counter()
        logits = self.engine.step(entries)
        self.trace.append([(r.index, n) for r, n in planned])
        self.stats.steps += 1
        for r, n in planned:
            self.stats.tokens += n
            if n == 1 and r.n_fed > 0 and r.n_fed + 1 == len(r.prompt) + len(r.generated) and r.generated:
                self.stats.decode_tokens += 1
            else:
                self.stats.prefill_tokens += n
            r.n_fed += n
        if samplers:
            new = self.sampler.sample(logits, [r.sampling for r in samplers], [r.index for r in samplers],
                                      [len(r.generated) for r in samplers])
            for r, tok in zip(samplers, new):
                r.generated.append(int(tok))
                if int(tok) in self.eos_set:
                    r.stop_reason = int(tok)
                    r.finished = True
                elif len(r.generated) >= r.budget:
                    r.finished = True
                if r.finished:
                    self.engine.release(r.handle)
                    r.handle = None
                    self.running.remove(r)
                    finished_now.append(r)
        if pure_decode:
            self.stats.decode_steps += 1
            self.stats.decode_step_tokens += len(planned)
            self.stats.decode_seconds += time.perf_counter() - t0
        return finished_now

    def run(self, requests: Sequence[Request]) -> Sequence[Request]:
        """Run the requests to completion; they are finished in place."""
        for r in requests:
            self.add(r)
        while self.has_work():
            self.step()
        return requests
