"""Continuous batching above the step function.

Each call of :meth:`Scheduler.step` builds ONE mixed batch under a token
budget: first one token for every running request that is decoding, then
portions of prompts (of running requests whose prompt is not through yet, then
of newly admitted ones, in arrival order), runs it, samples where a request's
last fed token was its newest, and finishes and frees at once.

Reference (src/scheduler/scheduler.cpp): per iteration it sweeps finished
requests (:73-107), admits whole prompts into a padding bucket (:114-155), runs
a padded all-prompt forward (:164-264) and then a second, all-decode forward
(:269-333); prompts are never split; it throws "OOM during decode" when the pool
is empty (:286-289); it samples greedily whatever the request asked (:233,
:310-312); ``max_new_tokens = 1`` yields two tokens because decode follows
prefill in the same iteration.  Decisions taken here instead:

* admission is FIFO; a request is admitted when a state slot is free and the
  pages for its first portion are free;
* pages run out during decode: the most recently admitted running request is
  preempted - its pages and slot go back, it returns to the FRONT of the
  waiting queue with its generated tokens kept, and is recomputed as a prompt
  of (prompt + generated) - until the rest fits; a request that cannot fit even
  alone finishes with reason ``kv_capacity``;
* ``max_new_tokens`` is exact; finish reasons are ``stop``, ``length``,
  ``max_context``, ``prompt_too_long`` and ``kv_capacity``.
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..cache.pages import OutOfPages
from ..sampling.params import SamplingParams
from .request import Request, RequestState
from .step import StepEntry


@dataclass
class SchedulerConfig:
    """``max_tokens_per_step``: token budget of a batch.  ``max_running``: most requests in
    flight (the reference has ``max_prefill_batch = 8`` and an unenforced ``max_decode_batch = 64``,
    src/scheduler/scheduler.h:38-44).  ``prefill_chunk``: longest portion of one prompt per step
    (0 = the budget)."""

    max_tokens_per_step: int = 2048
    max_running: int = 64
    prefill_chunk: int = 0
    max_context: int = 2048


@dataclass
class IterationStats:
    """Counterpart of the reference's per-step record (src/scheduler/scheduler.h:50-63)."""

    step: int = 0
    num_tokens: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    running: int = 0
    waiting: int = 0
    finished: int = 0
    preempted: int = 0
    free_pages: Tuple[int, ...] = ()
    seconds: float = 0.0


class Scheduler:
    """``executor`` provides ``cache`` (a CacheManager), ``add_request(rid)``, ``release(rid)`` and
    ``run(entries, sample_for) -> {rid: token}`` which runs one step and returns a sampled token
    for every request in ``sample_for`` (a list of Request)."""

    def __init__(self, executor, config: SchedulerConfig):
        self.ex = executor
        self.cfg = config
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self.history: List[IterationStats] = []
        self._admitted = 0
        self._steps = 0
        self.num_preemptions = 0

    # ------------------------------------------------------------------ #
    def submit(self, req: Request) -> None:
        if len(req.prompt) >= self.cfg.max_context:
            # the reference drops such a request as "prompt_too_long" (scheduler.cpp:120-131)
            req.finish("prompt_too_long")
            self.finished.append(req)
            return
        self.waiting.append(req)

    def done(self) -> bool:
        return not self.waiting and not self.running

    def drain_finished(self) -> List[Request]:
        out, self.finished = self.finished, []
        return out

    # ------------------------------------------------------------------ #
    def _preempt(self, victim: Request) -> None:
        self.ex.release(victim.rid)
        self.running.remove(victim)
        victim.num_computed = 0
        victim.state = RequestState.WAITING
        victim.metrics.preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(victim)

    def _finish(self, req: Request, reason: str) -> None:
        if req in self.running:
            self.ex.release(req.rid)
            self.running.remove(req)
        req.finish(reason)
        self.finished.append(req)

    def _pages_short(self, plan: List[Tuple[Request, int]]) -> bool:
        """Would the pools run dry if every (request, n tokens) of ``plan`` were reserved?"""
        cache = self.ex.cache
        need = [0] * len(cache.pools)
        for req, n in plan:
            for g, k in enumerate(cache.pages_needed(req.rid, n)):
                need[g] += k
        return any(k > pool.num_free for k, pool in zip(need, cache.pools))

    def plan(self) -> Tuple[List[Tuple[Request, int]], int]:
        """Decide the batch of this step: ``[(request, n tokens)]`` and how many were preempted."""
        preempted = 0
        while True:
            plan, p = self._plan_once(allow_admission=(preempted == 0))
            preempted += p
            if plan or not self.running:
                return plan, preempted
            # requests are running but none can take a single token: the pool is exhausted by
            # half-fed prompts.  Make room the same way as for decoding.
            victim = max(self.running, key=lambda r: r.admit_order)
            if len(self.running) == 1:
                self._finish(victim, "kv_capacity")
            else:
                self._preempt(victim)
                preempted += 1

    def _plan_once(self, allow_admission: bool) -> Tuple[List[Tuple[Request, int]], int]:
        cfg, cache = self.cfg, self.ex.cache
        preempted = 0
        # 1. one token for every decoding request; preempt from the back until they fit
        while True:
            decoding = [r for r in self.running if r.remaining == 1]
            plan = [(r, 1) for r in decoding]
            if not self._pages_short(plan):
                break
            victim = max(self.running, key=lambda r: r.admit_order)
            if len(self.running) == 1:
                self._finish(victim, "kv_capacity")
            else:
                self._preempt(victim)
                preempted += 1
        budget = cfg.max_tokens_per_step - len(plan)
        if budget < 0:
            plan = plan[:cfg.max_tokens_per_step]
            budget = 0
        chunk_cap = cfg.prefill_chunk or cfg.max_tokens_per_step

        def portion_that_fits(req: Request, want: int) -> int:
            n = want
            while n > 0 and self._pages_short(plan + [(req, n)]):
                # largest portion the free pages allow: shrink to the previous page boundary
                n = min(n - 1, ((cache.num_tokens(req.rid) + n - 1) // cache.page_size) * cache.page_size
                        - cache.num_tokens(req.rid))
            return max(n, 0)

        # 2. portions for running requests whose prompt is not through yet, oldest first
        for r in sorted(self.running, key=lambda r: r.admit_order):
            if budget <= 0:
                break
            if r.remaining > 1:
                n = portion_that_fits(r, min(r.remaining, budget, chunk_cap))
                if n > 0:
                    plan.append((r, n))
                    budget -= n
        # 3. admit new requests in arrival order
        while allow_admission and preempted == 0 and self.waiting and budget > 0 \
                and len(self.running) < cfg.max_running and cache.slots.num_free > 0:
            r = self.waiting[0]
            self.ex.add_request(r.rid)
            n = portion_that_fits(r, min(r.remaining, budget, chunk_cap))
            if n == 0:
                self.ex.release(r.rid)
                if not self.running and not plan:
                    # nothing else holds pages: this request can never start
                    self.waiting.popleft()
                    r.finish("kv_capacity")
                    self.finished.append(r)
                    continue
                break
            self.waiting.popleft()
            r.state = RequestState.RUNNING
            r.admit_order = self._admitted
            self._admitted += 1
            self.running.append(r)
            plan.append((r, n))
            budget -= n
        return plan, preempted

    def step(self) -> IterationStats:
        t0 = time.perf_counter()
        plan, preempted = self.plan()
        stats = IterationStats(step=self._steps, preempted=preempted)
        self._steps += 1
        if plan:
            entries, sample_for = [], []
            for r, n in plan:
                last = r.num_computed + n == r.num_tokens
                entries.append(StepEntry(r.rid, r.next_tokens(n), [n - 1] if last else []))
                if last:
                    sample_for.append(r)
                if n == 1 and r.remaining == 1:
                    stats.decode_tokens += 1
                else:
                    stats.prefill_tokens += n
            # If nothing but a stop token can change the batch, the next step decodes one token for
            # exactly these requests: an executor that can do so launches it ahead.
            ahead = (getattr(self.ex, "lookahead_capable", False) and len(sample_for) == len(self.running)
                     and not self.waiting
                     and all(len(r.generated) + 1 < r.params.max_new_tokens
                             and r.num_tokens + 1 < self.cfg.max_context for r in sample_for))
            try:
                tokens = self.ex.run(entries, sample_for, lookahead=True) if ahead \
                    else self.ex.run(entries, sample_for)
            except OutOfPages:
                # cannot happen if plan() counted right; treat as capacity failure of the newest request
                victim = max((r for r, _ in plan), key=lambda r: r.admit_order)
                self._finish(victim, "kv_capacity")
                return stats
            now = time.perf_counter()
            for r, n in plan:
                r.num_computed += n
                r.metrics.steps += 1
            for r in sample_for:
                tok = int(tokens[r.rid])
                r.generated.append(tok)
                if r.metrics.first_token is None:
                    r.metrics.first_token = now
                if tok in r.params.stop_token_ids:
                    self._finish(r, "stop")
                elif len(r.generated) >= r.params.max_new_tokens:
                    self._finish(r, "length")
                elif r.num_tokens >= self.cfg.max_context:
                    self._finish(r, "max_context")
            stats.num_tokens = stats.prefill_tokens + stats.decode_tokens
        stats.running = len(self.running)
        stats.waiting = len(self.waiting)
        stats.finished = len(self.finished)
        stats.free_pages = tuple(self.ex.cache.free_pages())
        stats.seconds = time.perf_counter() - t0
        self.history.append(stats)
        return stats

    def run_until_done(self, max_steps: int = 1 << 30) -> List[Request]:
        """Reference: ``run_until_done(max_iters)`` (src/scheduler/scheduler.cpp:373-379)."""
        out: List[Request] = []
        steps = 0
        while not self.done() and steps < max_steps:
            before = (len(self.running), len(self.waiting), len(self.finished))
            st = self.step()
            steps += 1
            out.extend(self.drain_finished())
            if st.num_tokens == 0 and (len(self.running), len(self.waiting), len(self.finished)) == before \
                    and st.preempted == 0:
                raise RuntimeError("Scheduler: no progress is possible (no tokens scheduled, nothing finished)")
        out.extend(self.drain_finished())
        return out
