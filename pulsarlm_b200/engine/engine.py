"""The Python entry point: Engine, submit / step / generate, and `complete`.

    engine = Engine("path/to/model", dtype="bfloat16", kv_cache_gib=4.0)
    outputs = engine.generate([[1, 2, 3]], SamplingParams(temperature=0.7, seed=1), max_tokens=16)

Option names and meanings follow the reference where it has them
(pulsarlm/src/pulsarlm/cli/__init__.py:179-238: dtype, kv_cache_gib,
prefill_tokens_per_step; pulsarlm/src/pulsarlm/core/engine.pyi:395-410:
submit(tokens, sampling=, max_tokens=) returning a request with take() and
cancel(); pulsarlm/src/pulsarlm/completion.py:43-109: complete()).
"""

from __future__ import annotations

import itertools
import sys
from typing import Iterator

import torch

from ..cache.manager import CacheManager, cache_bytes
from ..kernels import ops
from ..models.model import Model
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .loading import load_model, parse_dtype, random_model
from .runner import ModelRunner, StepEntry
from .scheduler import FROM_DEVICE, PlannedEntry, Request, Scheduler

DEFAULT_PAGE_SIZE = 16


class _Flight:
    """A step that has left for the device and whose sampled ids have not been read yet."""

    def __init__(self, entries: list[PlannedEntry], ids: torch.Tensor | None, pending, logits=None):
        self.entries = entries
        self.ids = ids          # int32 on the device: the tokens drawn, in the order of the entries that sample
        self.pending = pending  # their copy to the host (wait() gives them), or None when nothing samples
        self.logits = logits    # with record_logits: the rows the ids were drawn from
        samplers = [e for e in entries if e.samples]
        self.samplers = samplers
        self.row = {e.request.id: i for i, e in enumerate(samplers)}
        # A request that is preempted while the step runs has nothing to record when it ends.
        self.epochs = {e.request.id: e.request.preemptions for e in entries}


class _PendingCopy:
    """Token ids (and the kernels' status word behind them) on their way to the host."""

    def __init__(self, host: torch.Tensor, event: torch.cuda.Event, runner):
        self._host, self._event, self._runner = host, event, runner

    def wait(self) -> list[int]:
        self._event.synchronize()  # the step's one synchronisation
        values = self._host.tolist()
        if values[-1]:
            self._runner.raise_status(values[-1])
        return values[:-1]


def pages_for_bytes(needs: list, page_size: int, max_requests: int, dtype: torch.dtype, step_tokens: int,
                    budget: int) -> int:
    """The largest n_pages whose cache fits `budget` bytes: groups that keep every key get
    n_pages pages each, groups with a window at most what their requests can hold."""
    def total(n: int) -> int:
        return cache_bytes(needs, n, page_size, step_tokens, max_requests, dtype)

    low, high = 1, 2
    while total(high) <= budget and total(high) > total(low) and high < 1 << 30:
        low, high = high, high * 2
    while high - low > 1:
        mid = (low + high) // 2
        if total(mid) <= budget:
            low = mid
        else:
            high = mid
    return low


class Engine:
    def __init__(self, model, dtype="bfloat16", device="cuda:0", kv_cache_gib: float = 4.0,
                 page_size: int = DEFAULT_PAGE_SIZE, prefill_tokens_per_step: int = 256,
                 max_requests: int = 64, n_pages: int | None = None, stop_ids=None, seed: int | None = None,
                 cuda_graphs: bool = True, attention_mass_decay: float | None = None, lookahead: bool = True,
                 record_logits: bool = False):
        """model: a model folder, a built Model, or a config.json dict (random
        weights from `seed`). kv_cache_gib sizes the page pools unless n_pages
        gives the number of pages outright. stop_ids default to config.json's
        eos_token_id. attention_mass_decay: measure per-page attention mass with this
        decay (see CacheManager). The tensor-core kernels measure it themselves (captured
        decode steps, and prompt portions at pages of 16 to 64 tokens); single tokens of
        eager steps and shapes those kernels do not take attend on the CUDA-core kernel.
        lookahead: pipeline steps one deep (see step()). record_logits: keep, for
        every generated token, the fp32 logits row it was drawn from in
        `request.logits` (host tensors; for inspection and tests, it costs a copy of
        [vocab] floats per token)."""
        ops.require_device()
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.dtype = parse_dtype(dtype)
        if isinstance(model, Model):
            self.model = model
            self.dtype = model.ctx.dtype
        elif isinstance(model, dict):
            self.model = random_model(model, 0 if seed is None else seed, self.dtype, self.device)
        else:
            self.model = load_model(str(model), self.dtype, self.device)
        needs = self.model.cache_needs()
        # The scheduler gives a request at most prefill_tokens_per_step tokens a step, so a layer
        # group with a window needs only the pages that max_requests such requests can hold.
        step_tokens = max(1, int(prefill_tokens_per_step))
        if n_pages is None:
            n_pages = pages_for_bytes(needs, page_size, max_requests, self.dtype, step_tokens,
                                      int(kv_cache_gib * (1 << 30)))
        self.cache = CacheManager(needs, page_size, n_pages, max_requests, self.dtype, self.device,
                                  mass_decay=attention_mass_decay, step_tokens=step_tokens)
        self.runner = ModelRunner(self.model, self.cache)
        self.runner._bind()
        # Said once: a shape that the fast kernels do not take still runs, only slower.
        notes = sorted({note for part in self.model.parts()
                        for note in [getattr(part, "slow_path_note", lambda: None)()] if note})
        for note in notes:
            print(f"[pulsarlm_b200] note: {note}", file=sys.stderr, flush=True)
        self.sampler = Sampler(self.device)
        stops = self.model.spec.eos_token_ids if stop_ids is None else stop_ids
        self.scheduler = Scheduler(self.cache, stops, prefill_tokens_per_step)
        self.cuda_graphs = cuda_graphs and self.runner.graphs_allowed
        self.lookahead = lookahead
        self.record_logits = record_logits
        self._inflight: _Flight | None = None
        self._host_ids: list[torch.Tensor] | None = None
        self._host_turn = 0
        self._ids = itertools.count()
        self.vocab_size = self.model.spec.vocab_size

    # ------------------------------------------------------------------ requests
    def submit(self, tokens: list[int], *, sampling: SamplingParams | None = None, max_tokens: int | None = None,
               ignore_eos: bool = False) -> Request:
        """Queues a request; it advances as `step()` is called. Token ids are
        validated here (pulsarlm-core/src/engine/engine.cpp:57-87)."""
        tokens = [int(t) for t in tokens]
        if not tokens:
            raise ValueError("a request needs at least one token")
        bad = [t for t in tokens if not 0 <= t < self.vocab_size]
        if bad:
            raise ValueError(f"token id {bad[0]} is outside [0, {self.vocab_size})")
        sampling = sampling or SamplingParams()
        request = Request(next(self._ids), tokens, sampling, max_tokens, ignore_eos, seed=sampling.resolved_seed())
        self.scheduler.add(request)
        return request

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    def step(self) -> list[Request]:
        """Advances the engine by one scheduler step on the GPU; returns the requests
        that ended.

        With `lookahead` steps are pipelined one deep: the call launches a step and
        returns; the next call first plans and launches the step after it, and only then
        reads the earlier step's token ids. The host's work for a step thus overlaps the
        GPU's, and a request's output lags its step by one call. The later step is planned
        as if every request of the earlier one went on (unless the token being drawn is
        certain to be its last): their tokens are taken on the device from the ids the
        earlier step is still drawing. A request that then ends on a stop token has
        computed one token too many, which is dropped."""
        flight = self._inflight
        entries, ended = self.scheduler.plan()
        launched = self._launch(entries, flight) if entries else None  # (if this raises, `flight` stays to be read)
        self._inflight = None
        done = self._settle(flight) if flight is not None else []
        if launched is not None:
            if self.lookahead:
                self._inflight = launched
            else:
                done = done + self._settle(launched)
        return done + ended

    def _launch(self, entries: list[PlannedEntry], earlier: "_Flight | None") -> "_Flight":
        """Launches the planned entries (a captured decode step when all are single tokens
        that sample, else an eager step), starts the copy of the drawn ids to the host
        and tells the scheduler that the step has left."""
        taken = None
        if any(e.tokens == [FROM_DEVICE] for e in entries):
            rows = [earlier.row[e.request.id] if e.tokens == [FROM_DEVICE] else -1 for e in entries]
            taken = (earlier.ids, rows)
        step_entries = [StepEntry(e.request.id, e.tokens if e.tokens != [FROM_DEVICE] else [0],
                                  [len(e.tokens) - 1] if e.samples else []) for e in entries]
        samplers = [e for e in entries if e.samples]
        sampling = [e.request.sampling for e in samplers]
        seeds = [e.request.seed for e in samplers]
        counts = [e.request.draw_count for e in samplers]
        if self.cuda_graphs and len(samplers) == len(entries) and all(
                len(e.tokens) == 1 and e.request.max_tokens != 0 for e in entries):
            ids = self.runner.decode_step(step_entries, sampling, seeds, counts, taken=taken)
            graph = self.runner.last_graph
            kept = graph.logits[: len(entries)].clone() if self.record_logits else None  # (the next replay overwrites them)
            flight = _Flight(entries, ids, graph.read_back(), kept)
        else:
            logits = self.runner.step(step_entries, taken=taken)
            ids = pending = None
            if samplers and logits is not None:
                ids = self.sampler.sample(logits, sampling, seeds, counts).to(torch.int32)
                pending = self._read_back(ids)
            flight = _Flight(entries, ids, pending, logits if self.record_logits else None)
        self.scheduler.advance(entries)
        return flight

    def _read_back(self, ids: torch.Tensor) -> _PendingCopy:
        """Starts the copy of an eager step's ids to the host, the kernels' status word
        behind them. Two pinned buffers alternate: one earlier result may still be unread."""
        n = ids.numel()
        if self._host_ids is None or self._host_ids[0].numel() < n + 1:
            size = max(n + 1, self.cache.max_requests + 1)
            self._host_ids = [torch.empty(size, dtype=torch.int32, pin_memory=True) for _ in range(2)]
            self._host_events = [torch.cuda.Event(), torch.cuda.Event()]
        turn, self._host_turn = self._host_turn, self._host_turn ^ 1
        host = self._host_ids[turn][: n + 1]
        host.copy_(torch.cat([ids, self.runner.status]), non_blocking=True)
        self._host_events[turn].record()
        return _PendingCopy(host, self._host_events[turn], self.runner)

    def _settle(self, flight: "_Flight") -> list[Request]:
        """Reads a launched step's ids and records them; returns the requests that ended."""
        host = flight.pending.wait() if flight.pending is not None else []
        sampled = {e.request.id: t for e, t in zip(flight.samplers, host)}
        before = None
        if self.record_logits and flight.logits is not None:
            before = [len(e.request.output) for e in flight.samplers]
        done = self.scheduler.settle(flight.entries, sampled, flight.epochs)
        if before is not None:
            rows = flight.logits[: len(flight.samplers)].float().cpu()
            for e, had, row in zip(flight.samplers, before, rows):
                if len(e.request.output) > had:
                    e.request.logits.append(row)
        return done

    def sync(self) -> list[Request]:
        """Reads a step still in flight; returns the requests that ended in it."""
        flight, self._inflight = self._inflight, None
        return self._settle(flight) if flight is not None else []

    # ------------------------------------------------------------------ whole runs
    def generate(self, prompts: list[list[int]], sampling=None, max_tokens: int | None = 16,
                 ignore_eos: bool = False) -> list[list[int]]:
        """Generated token ids for each prompt (host lists in, host lists out).
        `sampling`: one SamplingParams for all, or one per prompt."""
        if isinstance(sampling, (list, tuple)):
            if len(sampling) != len(prompts):
                raise ValueError("one SamplingParams per prompt")
            per_prompt = list(sampling)
        else:
            per_prompt = [sampling] * len(prompts)
        requests = [self.submit(p, sampling=s, max_tokens=max_tokens, ignore_eos=ignore_eos)
                    for p, s in zip(prompts, per_prompt)]
        while any(not r.finished for r in requests):
            self.step()
        self.runner.check_status()
        failed = [r for r in requests if r.finish_reason == "oom"]
        if failed:
            raise MemoryError(f"{len(failed)} request(s) did not fit the KV cache even alone "
                              f"({self.cache.n_pages} pages of {self.cache.page_size} tokens)")
        return [list(r.output) for r in requests]

    def stats(self) -> dict:
        return {"steps": self.runner.steps, "tokens_run": self.runner.tokens_run,
                "preemptions": self.scheduler.preemptions, "cache": self.cache.stats()}


def complete(engine: Engine, prompt_ids: list[int], *, sampling: SamplingParams | None = None,
             max_tokens: int | None = None) -> Iterator[int]:
    """Yields a request's tokens as they are generated (the synchronous counterpart
    of the reference's `complete`, pulsarlm/src/pulsarlm/completion.py:43-109).
    Closing the generator early cancels the request."""
    request = engine.submit(prompt_ids, sampling=sampling, max_tokens=max_tokens)
    try:
        while not request.finished:
            engine.step()
            yield from request.take()
        yield from request.take()
        if request.finish_reason == "oom":
            raise MemoryError("the request did not fit the KV cache")
    finally:
        if not request.finished:
            request.cancel()
            engine.step()
