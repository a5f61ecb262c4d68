"""The scheduler: which requests run in the next step, with how many tokens each.

Decisions, all deterministic:

* Admission: requests wait in arrival order; the first waiting request is admitted
  when a slot is free and the pages of its first portion are free. (The reference
  has no queue: a request that finds no room ends with `oom`,
  pulsarlm-core/src/engine/scheduler.cpp:36-52, executor.cpp:477-483.)
* Composition of a step: every decoding request runs its one token; then prompts
  are cut into portions that share `prefill_tokens_per_step` in admission order
  (scheduler.cpp:77-107). A request samples in a step only if the step consumes
  all its pending tokens.
* Finishing: a sampled stop id (unless `ignore_eos`) or `max_tokens` generated
  tokens end the request; `max_tokens = 0` runs the prompt and ends
  (executor.cpp:801-811). Its pages and slot are given back at once.
* Pages run out: the most recently admitted running request is preempted: its
  pages and slot are given back, and it returns to the front of the waiting
  queue with prompt + generated tokens as its new prompt (recomputed later; the
  tokens it goes on to draw are unchanged, since draws are keyed by seed and draw
  count). A request that cannot get its pages even when it is the only one running
  ends with the error `oom`. (The reference ends the request that could not grow,
  executor.cpp:862-870.)

The scheduler only does bookkeeping against the cache manager; the caller runs
the model on what `plan()` returns and reports sampled tokens to `finish_step()`.
"""

from __future__ import annotations

import dataclasses
from collections import deque

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams


@dataclasses.dataclass
class Request:
    """One generation request and its progress."""

    id: object
    prompt: list[int]
    sampling: SamplingParams = dataclasses.field(default_factory=SamplingParams)
    max_tokens: int | None = None
    ignore_eos: bool = False
    # progress
    seed: int = 0
    output: list[int] = dataclasses.field(default_factory=list)
    pending: list[int] = dataclasses.field(default_factory=list)
    taken: int = 0
    state: str = "waiting"  # waiting | running | finished
    finish_reason: str | None = None  # stop | length | cancelled | oom
    cancelled: bool = False
    preemptions: int = 0

    def take(self) -> list[int]:
        """Tokens generated since the last take()."""
        new = self.output[self.taken:]
        self.taken = len(self.output)
        return new

    def cancel(self) -> None:
        self.cancelled = True

    @property
    def finished(self) -> bool:
        return self.state == "finished"

    @property
    def draw_count(self) -> int:
        return len(self.output)


@dataclasses.dataclass
class PlannedEntry:
    request: Request
    tokens: list[int]
    samples: bool


class Scheduler:
    def __init__(self, cache: CacheManager, stop_ids=(), prefill_tokens_per_step: int = 256,
                 max_step_entries: int | None = None):
        if prefill_tokens_per_step <= 0:
            raise ValueError("prefill_tokens_per_step must be positive")
        self.cache = cache
        self.stop_ids = frozenset(int(s) for s in stop_ids)
        self.prefill_tokens_per_step = prefill_tokens_per_step
        self.max_step_entries = max_step_entries or cache.max_requests
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []  # admission order
        self.preemptions = 0

    # ------------------------------------------------------------------ intake
    def add(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError(f"request {request.id!r}: the prompt is empty")
        if request.max_tokens is not None and request.max_tokens < 0:
            raise ValueError(f"request {request.id!r}: max_tokens must be >= 0")
        request.pending = list(request.prompt)
        request.state = "waiting"
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ ending
    def _finish(self, request: Request, reason: str) -> None:
        if self.cache.is_open(request.id):
            self.cache.close(request.id)
        if request in self.running:
            self.running.remove(request)
        request.state = "finished"
        request.finish_reason = reason
        request.pending = []

    def _preempt(self, request: Request) -> None:
        """Back to the front of the queue; everything it computed is recomputed later."""
        self.cache.close(request.id)
        self.running.remove(request)
        request.pending = list(request.prompt) + list(request.output)
        request.state = "waiting"
        request.preemptions += 1
        self.preemptions += 1
        self.waiting.appendleft(request)

    def _drop_cancelled(self) -> list[Request]:
        ended = []
        for request in [r for r in self.running if r.cancelled]:
            self._finish(request, "cancelled")
            ended.append(request)
        for request in [r for r in self.waiting if r.cancelled]:
            self.waiting.remove(request)
            self._finish(request, "cancelled")
            ended.append(request)
        return ended

    # ------------------------------------------------------------------ planning
    def _reserve(self, request: Request, count: int, protected: set) -> bool:
        """Pages for `count` more tokens of a running request, preempting the newest
        other running request (never one in `protected`) while that helps."""
        new_len = self.cache.length(request.id) + count
        while not self.cache.reserve(request.id, new_len):
            victims = [r for r in self.running if r is not request and id(r) not in protected]
            if not victims:
                return False
            self._preempt(victims[-1])
        return True

    def plan(self) -> tuple[list[PlannedEntry], list[Request]]:
        """The next step's entries (decode entries first, then prompt portions), and
        the requests that ended while planning (cancelled, or out of memory)."""
        ended = self._drop_cancelled()
        entries: list[PlannedEntry] = []
        planned: set = set()

        # 1. decoding requests, oldest first; a preempted one simply leaves `running`.
        for request in list(self.running):
            if request not in self.running or len(request.pending) != 1:
                continue
            if len(entries) >= self.max_step_entries:
                break
            if self._reserve(request, 1, planned):
                entries.append(PlannedEntry(request, list(request.pending), True))
                planned.add(id(request))
            elif not planned and len(self.running) == 1:
                self._finish(request, "oom")
                ended.append(request)
            # else: it waits for a later step, holding what it has.

        # 2. prompt portions of running requests, then of newly admitted ones.
        budget = self.prefill_tokens_per_step
        for request in list(self.running):
            if budget == 0 or len(entries) >= self.max_step_entries:
                break
            if request not in self.running or len(request.pending) <= 1 or id(request) in planned:
                continue
            count = min(len(request.pending), budget)
            if self._reserve(request, count, planned):
                entries.append(PlannedEntry(request, request.pending[:count], count == len(request.pending)))
                planned.add(id(request))
                budget -= count
            elif not planned and len(self.running) == 1:
                self._finish(request, "oom")
                ended.append(request)

        while self.waiting and budget > 0 and len(entries) < self.max_step_entries:
            request = self.waiting[0]
            count = min(len(request.pending), budget)
            if self.cache.open(request.id) is None:
                break
            if not self.cache.reserve(request.id, count):
                self.cache.close(request.id)
                if not self.running:
                    # Alone and still too large for the pool: it can never run.
                    self.waiting.popleft()
                    self._finish(request, "oom")
                    ended.append(request)
                    continue
                break
            self.waiting.popleft()
            request.state = "running"
            self.running.append(request)
            # A lone token samples like a decode entry.
            entries.append(PlannedEntry(request, request.pending[:count], count == len(request.pending)))
            planned.add(id(request))
            budget -= count
        # Decode entries (one pending token) first, as the kernels' launchers like it.
        entries.sort(key=lambda e: 0 if len(e.tokens) == 1 else 1)
        return entries, ended

    # ------------------------------------------------------------------ after a step
    def finish_step(self, entries: list[PlannedEntry], sampled: dict) -> list[Request]:
        """Records a step: `sampled[request.id]` is the token drawn for each entry
        that samples. Returns the requests that finished."""
        ended = []
        for entry in entries:
            request = entry.request
            if request.state != "running":
                continue
            del request.pending[: len(entry.tokens)]
            if not entry.samples:
                continue
            if request.max_tokens == 0:
                self._finish(request, "length")
                ended.append(request)
                continue
            token = int(sampled[request.id])
            request.output.append(token)
            if token in self.stop_ids and not request.ignore_eos:
                self._finish(request, "stop")
                ended.append(request)
            elif request.max_tokens is not None and len(request.output) >= request.max_tokens:
                self._finish(request, "length")
                ended.append(request)
            else:
                request.pending = [token]
        return ended
