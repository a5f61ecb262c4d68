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
the model on what `plan()` returns and reports sampled tokens to `finish_step()`,
or in two halves: `advance()` when the step has left for the device and `settle()`
when its tokens have arrived. Between the two the next step can be planned: a
request that samples in the step under way is planned with the token being drawn
(`FROM_DEVICE` in its entry: the caller takes it from the earlier step's ids on the
device), unless that token is certain to be its last. A request that then stops on
a stop id has computed one token too many, which is dropped.
The decisions are made in C++ (SchedulerCore, pulsarlm_b200/csrc_host); the class
below keeps the Python-side Request objects and token lists in step with it.
"""

from __future__ import annotations

import ctypes
import dataclasses
from collections import deque

from ..cache.manager import CacheManager
from ..host import core
from ..sampling.params import SamplingParams


FROM_DEVICE = -1  # in an entry's tokens: the token a step still under way is drawing for this request


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
    unsettled: int = 0  # tokens being drawn by steps that have left and are not settled yet
    logits: list = dataclasses.field(default_factory=list)  # filled by an engine that records logits

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
        """How many tokens were drawn for the request before the one to draw next."""
        return len(self.output) + self.unsettled


@dataclasses.dataclass
class PlannedEntry:
    request: Request
    tokens: list[int]
    samples: bool


class Scheduler:
    """The Python face of the scheduler core (C++, class SchedulerCore in
    pulsarlm_b200/csrc_host/host_core.cpp), which makes the decisions above on
    counts alone; this class keeps the token lists and the Request objects in step
    with it."""

    def __init__(self, cache: CacheManager, stop_ids=(), prefill_tokens_per_step: int = 256,
                 max_step_entries: int | None = None):
        if prefill_tokens_per_step <= 0:
            raise ValueError("prefill_tokens_per_step must be positive")
        self.cache = cache
        self.prefill_tokens_per_step = prefill_tokens_per_step
        self.max_step_entries = max_step_entries or cache.max_requests
        self._lib = core.library()
        self._core = self._lib.plh_sched_create(cache.book, prefill_tokens_per_step, self.max_step_entries)
        self._requests: dict[int, Request] = {}  # by the cache's handle
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []  # admission order
        self.stop_ids = stop_ids
        self._counts = (ctypes.c_int32 * 3)()
        self._capacity = 0
        self._ensure_capacity(max(64, 2 * cache.max_requests))

    def _ensure_capacity(self, n: int) -> None:
        """Room in the buffers the core writes a plan into: a plan names each known
        request at most once as an entry, once as ended and once as preempted."""
        if n <= self._capacity:
            return
        n = max(n, 2 * self._capacity)
        self._capacity = n
        self._entries = (ctypes.c_int64 * (3 * n))()
        self._ended = (ctypes.c_int64 * (2 * n))()
        self._preempted = (ctypes.c_int64 * n)()
        self._tokens = (ctypes.c_int32 * n)()

    def __del__(self):
        if getattr(self, "_core", None):
            self._lib.plh_sched_destroy(self._core)
            self._core = None

    @property
    def stop_ids(self) -> frozenset:
        return self._stop_ids

    @stop_ids.setter
    def stop_ids(self, ids) -> None:
        self._stop_ids = frozenset(int(s) for s in ids)
        array = (ctypes.c_int32 * max(1, len(self._stop_ids)))(*sorted(self._stop_ids))
        self._lib.plh_sched_set_stop_ids(self._core, array, len(self._stop_ids))

    @property
    def preemptions(self) -> int:
        return self._lib.plh_sched_preemptions(self._core)

    # ------------------------------------------------------------------ intake
    def add(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError(f"request {request.id!r}: the prompt is empty")
        if request.max_tokens is not None and request.max_tokens < 0:
            raise ValueError(f"request {request.id!r}: max_tokens must be >= 0")
        handle = self.cache.handle(request.id)
        code = self._lib.plh_sched_add(self._core, handle, len(request.prompt),
                                       -1 if request.max_tokens is None else request.max_tokens,
                                       int(request.ignore_eos))
        if code != 0:
            raise ValueError(f"request {request.id!r} cannot be added twice")
        request.pending = list(request.prompt)
        request.state = "waiting"
        self._requests[handle] = request
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self._lib.plh_sched_has_work(self._core))

    # ------------------------------------------------------------------ mirroring the core
    def _end(self, handle: int, reason: str) -> Request:
        request = self._requests.pop(handle)
        if request in self.running:
            self.running.remove(request)
        elif request in self.waiting:
            self.waiting.remove(request)
        request.state = "finished"
        request.finish_reason = reason
        request.pending = []
        self.cache.forget(request.id)
        return request

    def plan(self) -> tuple[list[PlannedEntry], list[Request]]:
        """The next step's entries (single-token entries first, then prompt portions),
        and the requests that ended while planning (cancelled, or out of memory)."""
        for request in self._requests.values():
            if request.cancelled:
                self._lib.plh_sched_cancel(self._core, self.cache.handle(request.id))
        self._ensure_capacity(len(self._requests) + 1)
        code = self._lib.plh_sched_plan(self._core, self._entries, self._ended, self._preempted, self._capacity,
                                        self._counts)
        if code != 0:
            raise RuntimeError("the scheduler core planned more entries than fit its buffers")
        n_entries, n_ended, n_preempted = self._counts[0], self._counts[1], self._counts[2]
        for i in range(n_preempted):
            request = self._requests[self._preempted[i]]
            # Back to the front of the queue; everything it computed is recomputed later.
            if request in self.running:
                self.running.remove(request)
            request.pending = list(request.prompt) + list(request.output)
            request.unsettled = 0  # (a token still being drawn is dropped; it is drawn again later)
            request.state = "waiting"
            request.preemptions += 1
            self.waiting.appendleft(request)
        ended = [self._end(self._ended[2 * i], core.REASONS[self._ended[2 * i + 1]]) for i in range(n_ended)]
        entries = []
        for i in range(n_entries):
            request = self._requests[self._entries[3 * i]]
            count, samples = self._entries[3 * i + 1], bool(self._entries[3 * i + 2])
            if request.state == "waiting":  # admitted in this plan
                self.waiting.remove(request)
                self.running.append(request)
                request.state = "running"
                self.cache.zero_states(self.cache.slot(request.id))
            entries.append(PlannedEntry(request, request.pending[:count], samples))
        return entries, ended

    # ------------------------------------------------------------------ after a step
    def _flat(self, entries: list[PlannedEntry]):
        flat = (ctypes.c_int64 * (3 * max(1, len(entries))))()
        for i, entry in enumerate(entries):
            flat[3 * i] = self.cache.handle(entry.request.id)
            flat[3 * i + 1] = len(entry.tokens)
            flat[3 * i + 2] = int(entry.samples)
        return flat

    def advance(self, entries: list[PlannedEntry]) -> None:
        """The step has left for the device: its tokens are consumed, and a request that
        samples in it goes on with the token being drawn (`FROM_DEVICE`) unless that token
        is its last."""
        self._lib.plh_sched_advance(self._core, self._flat(entries), len(entries))
        for entry in entries:
            request = entry.request
            del request.pending[: len(entry.tokens)]
            if entry.samples and request.max_tokens != 0:
                request.unsettled += 1
                last = request.max_tokens is not None and request.draw_count >= request.max_tokens
                request.pending = [] if last else [FROM_DEVICE]

    def settle(self, entries: list[PlannedEntry], sampled: dict, epochs: dict | None = None) -> list[Request]:
        """The tokens of a step that `advance` saw: `sampled[request.id]` for each entry
        that samples. `epochs[request.id]`: the request's `preemptions` when the step left;
        an entry whose request was preempted or ended since has nothing to record. Returns
        the requests that finished."""
        entries = [e for e in entries if e.request.state == "running"
                   and (epochs is None or epochs.get(e.request.id) == e.request.preemptions)]
        for i, entry in enumerate(entries):
            request = entry.request
            token = int(sampled.get(request.id, 0)) if entry.samples else 0
            self._tokens[i] = token
            if entry.samples and request.max_tokens != 0:
                request.output.append(token)
                request.unsettled -= 1
                if request.unsettled == 0 and request.pending == [FROM_DEVICE]:
                    request.pending = [token]  # no later step has taken it from the device
        n_ended = self._lib.plh_sched_settle(self._core, self._flat(entries), self._tokens, len(entries), self._ended,
                                             self._capacity)
        return [self._end(self._ended[2 * i], core.REASONS[self._ended[2 * i + 1]]) for i in range(n_ended)]

    def finish_step(self, entries: list[PlannedEntry], sampled: dict) -> list[Request]:
        """Records a step at once: `sampled[request.id]` is the token drawn for each entry
        that samples. Returns the requests that finished."""
        entries = [e for e in entries if e.request.state == "running"]
        self.advance(entries)
        return self.settle(entries, sampled)
