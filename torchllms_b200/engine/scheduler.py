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
from typing import Deque, Iterable, List, Optional, Sequence, Set, Tuple

import torch

from ..cache.manager import OutOfPages
from ..sampling.sampler import Sampler, SamplingParams
from .step import Engine


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
    launched_ahead: int = 0          # decode steps put on the device before the step before them was read


@dataclass
class _Launched:
    """A step that is on the device."""

    planned: List[Tuple[Request, int]]
    samplers: List[Request]               # the requests that get a token from it, in row order
    on_device: Optional[torch.Tensor]     # their tokens, on the device
    tokens: object                        # the same on their way to the host (None: nobody samples)
    pure_decode: bool


class Scheduler:
    def __init__(self, engine: Engine, sampler: Sampler, *, max_num_seqs: Optional[int] = None,
                 max_num_batched_tokens: int = 2048, prefill_chunk: Optional[int] = None,
                 eos_ids: Iterable[int] = (), look_ahead: bool = True):
        self.engine = engine
        self.look_ahead = bool(look_ahead)
        self._in_flight: Optional[_Launched] = None   # a step on the device whose tokens are not read yet
        self._last_read = 0.0                          # when the last step's tokens reached the host
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
        need = len(request.prompt) + request.budget - 1   # the last sampled token is never fed
        most = min(self.engine.max_len, self._most_cached_tokens(need))
        if need > most:
            request.finished = True
            request.error = (f"request needs {need} cached tokens but the engine holds at most "
                             f"{most} for one request")
            return
        self.waiting.append(request)

    def _most_cached_tokens(self, need: int) -> int:
        """How long a request that has the pool to itself may grow, given that it wants ``need``.
        A group that keeps every key holds its page count times the page size.  A window group
        gives pages back as the request grows: it only has to hold the window and the portion
        being fed (plus a page for where they start and end), however long the request gets."""
        cache = self.engine.cache
        page = cache.page_size
        most = need
        for g in cache.groups:
            held = g.allocator.n_pages * page
            if g.need.kind == "window":
                portion = min(self.prefill_chunk, self.max_num_batched_tokens)
                if (-(-(g.need.window + portion) // page) + 1) * page <= held:
                    continue                      # it never holds more than that: no limit from this group
            most = min(most, held)
        return most

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
        """Complete one step (plan, run, sample, read back) and return the requests that finished
        in it.

        With ``look_ahead``, the next decode step is put on the device before this step's tokens
        are read: its token ids go from the sampler's output to the model's input on the device,
        so the device does not wait while the host reads tokens and books them.  That next step is
        a bet that no request ends on a stop token: a request that does has one row computed in
        vain (its pages are freed as usual; no other row depends on it).  Ending on the budget is
        known beforehand and is no bet.  A call still completes exactly one step."""
        # a step's time runs from this call's start, or, if it was launched during the call before,
        # from the moment that call had its tokens (the device went straight on to this one)
        started = self._last_read if self._in_flight is not None else time.perf_counter()
        finished_now: List[Request] = []
        current, self._in_flight = self._in_flight, None
        if current is None:
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
            current = self._launch(planned)
        if self.look_ahead and current.tokens is not None:
            self._in_flight = self._launch_ahead(current)
        if current.tokens is not None:
            new = self.sampler.finish(current.tokens)
            self._last_read = time.perf_counter()
            for r, tok in zip(current.samplers, new):
                if r.finished:
                    continue                    # it ended a step ago; this row was the lost bet
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
        if self._in_flight is not None and all(r.finished for r in self._in_flight.samplers):
            self._in_flight = None              # nobody is left to read it
        if current.pure_decode:
            self.stats.decode_steps += 1
            self.stats.decode_step_tokens += len(current.planned)
            self.stats.decode_seconds += time.perf_counter() - started
        return finished_now

    def _launch(self, planned: List[Tuple[Request, int]], device_tokens=None, rows=None, ahead: int = 0) -> "_Launched":
        """Put a planned step and its sampling on the device; nothing here waits for the device.
        ``ahead`` is 1 when the requests' last tokens are not on the host yet: they are rows
        ``rows`` of ``device_tokens``."""
        shape, tokens, samplers = [], [], []
        for r, n in planned:
            completes = r.n_fed + n == len(r.prompt) + len(r.generated) + ahead
            shape.append((r.handle, n, [n - 1] if completes else []))
            if completes:
                samplers.append(r)
            if device_tokens is None:
                tokens.extend(r.span(r.n_fed, n))
        pure_decode = all(n == 1 and r.n_fed > 0 and (r.generated or ahead) for r, n in planned)
        prepared = self.engine.prepare(shape)       # OutOfPages leaves everything as it was
        if device_tokens is None:
            logits = self.engine.run_prepared(prepared, tokens)
        else:
            logits = self.engine.run_prepared(prepared, device_tokens, rows)
        self.trace.append([(r.index, n) for r, n in planned])
        self.stats.steps += 1
        for r, n in planned:
            self.stats.tokens += n
            if (n == 1 and r.n_fed > 0 and r.n_fed + 1 == len(r.prompt) + len(r.generated) + ahead
                    and (r.generated or ahead)):
                self.stats.decode_tokens += 1
            else:
                self.stats.prefill_tokens += n
            r.n_fed += n
        pending = on_device = None
        if samplers:
            on_device = self.sampler.launch(logits, [r.sampling for r in samplers], [r.index for r in samplers],
                                            [len(r.generated) + ahead for r in samplers])
            pending = self.sampler.read_back(on_device)
        return _Launched(planned, samplers, on_device, pending, pure_decode)

    def _launch_ahead(self, current: "_Launched") -> Optional["_Launched"]:
        """The decode step after ``current`` for the requests that will still run if none of them
        stops on a token, launched before ``current``'s tokens are known; ``None`` when the next step
        needs a fresh plan (somebody waits for admission, a prompt is still being fed, pages ran out)."""
        if self.waiting and len(self.running) < self.max_num_seqs:
            return None
        place = {id(r): i for i, r in enumerate(current.samplers)}
        if any(id(r) not in place for r in self.running):
            return None
        # whoever has room for another token after the one being sampled now
        stay = [r for r in self.running if len(r.generated) + 1 < r.budget]
        if not stay or len(stay) > self.max_num_batched_tokens:
            return None
        try:
            launched = self._launch([(r, 1) for r in stay], device_tokens=current.on_device,
                                    rows=[place[id(r)] for r in stay], ahead=1)
        except OutOfPages:
            return None                         # the ordinary plan decides whom to pre-empt
        self.stats.launched_ahead += 1
        return launched

    def run(self, requests: Sequence[Request]) -> Sequence[Request]:
        """Run the requests to completion; they are finished in place."""
        for r in requests:
            self.add(r)
        while self.has_work():
            self.step()
        return requests
