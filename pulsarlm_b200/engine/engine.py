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
from .scheduler import PlannedEntry, Request, Scheduler

DEFAULT_PAGE_SIZE = 16


class _Flight:
    """A decode step that was launched and whose sampled ids have not been read yet."""

    def __init__(self, entries: list[PlannedEntry], ids: torch.Tensor, pending, logits=None):
        self.entries = entries
        self.ids = ids          # int32 [entries] on the device
        self.pending = pending  # their copy to the host
        self.logits = logits    # with record_logits: a copy of the rows the ids were drawn from


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
        lookahead: pipeline decode steps one deep (see step()). record_logits: keep, for
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
        self.lookahead = lookahead and self.cuda_graphs
        self.record_logits = record_logits
        self._inflight: _Flight | None = None
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

        Steps made of single decode tokens are pipelined one deep (`lookahead`): the
        call launches the step and returns; the next call first launches the step
        after it, whose tokens the GPU takes from the ids the earlier step is still
        sampling, and only then reads the earlier step's ids. The host's work for a
        step thus overlaps the GPU's, and a request's output lags its step by one
        call. The step after is launched early only when it is certain to be the same
        requests again (nobody waiting or cancelled, nobody at its token limit, pages
        to spare); a request that ends on a stop token has then computed one token too
        many, which is dropped."""
        done: list[Request] = []
        flight = self._inflight
        if flight is not None:
            self._inflight = None
            if self._can_look_ahead(flight):
                entries, ended = self.scheduler.plan()
                same = not ended and len(entries) == len(flight.entries) and all(
                    e.request is f.request and len(e.tokens) == 1 and e.samples
                    for e, f in zip(entries, flight.entries))
                if same:
                    ahead = self._launch_decode(entries, device_tokens=flight.ids, count_offset=1)
                    done = self._finish(flight)
                    self._inflight = ahead
                    return done
                # (not expected under the conditions checked) finish, then run what was planned
                done = self._finish(flight)
                entries = [PlannedEntry(e.request, e.request.pending[: len(e.tokens)], e.samples)
                           for e in entries if e.request.state == "running"]
                return done + ended + self._execute(entries)
            done = self._finish(flight)
        entries, ended = self.scheduler.plan()
        return done + ended + self._execute(entries)

    def _execute(self, entries: list[PlannedEntry]) -> list[Request]:
        """Runs planned entries; returns the requests that ended (none yet when the step
        stays in flight)."""
        if not entries:
            return []
        if self.cuda_graphs and all(len(e.tokens) == 1 and e.samples and e.request.max_tokens != 0
                                    for e in entries):
            flight = self._launch_decode(entries)
            if self.lookahead:
                self._inflight = flight
                return []
            return self._finish(flight)
        step_entries = [StepEntry(e.request.id, e.tokens, [len(e.tokens) - 1] if e.samples else [])
                        for e in entries]
        sampled: dict = {}
        samplers = [e for e in entries if e.samples]
        logits = self.runner.step(step_entries)
        if samplers and logits is not None:
            drawn = self.sampler.sample(
                logits, [e.request.sampling for e in samplers], [e.request.seed for e in samplers],
                [e.request.draw_count for e in samplers])
            # the step's one synchronisation; the kernels' status word rides along
            host = torch.cat([drawn.to(torch.int32), self.runner.status]).cpu().tolist()
            if host[-1]:
                self.runner.raise_status(host[-1])
            sampled = {e.request.id: t for e, t in zip(samplers, host)}
            return self._record(samplers, sampled, logits, entries)
        return self.scheduler.finish_step(entries, sampled)

    def _record(self, samplers: list[PlannedEntry], sampled: dict, logits, entries=None) -> list[Request]:
        """finish_step, and with record_logits the rows of the tokens that were kept."""
        before = [len(e.request.output) for e in samplers] if self.record_logits else None
        done = self.scheduler.finish_step(samplers if entries is None else entries, sampled)
        if self.record_logits and logits is not None:
            rows = logits[: len(samplers)].float().cpu()
            for e, had, row in zip(samplers, before, rows):
                if len(e.request.output) > had:
                    e.request.logits.append(row)
        return done

    def _launch_decode(self, entries: list[PlannedEntry], device_tokens: torch.Tensor | None = None,
                       count_offset: int = 0) -> "_Flight":
        step_entries = [StepEntry(e.request.id, e.tokens, [0]) for e in entries]
        ids = self.runner.decode_step(
            step_entries, [e.request.sampling for e in entries], [e.request.seed for e in entries],
            [e.request.draw_count + count_offset for e in entries], device_tokens=device_tokens)
        graph = self.runner.last_graph
        kept = graph.logits[: len(entries)].clone() if self.record_logits else None  # the next replay overwrites them
        return _Flight(entries, ids, graph.read_back(), kept)

    def _finish(self, flight: "_Flight") -> list[Request]:
        host = flight.pending.wait()
        return self._record(flight.entries, {e.request.id: t for e, t in zip(flight.entries, host)}, flight.logits)

    def _can_look_ahead(self, flight: "_Flight") -> bool:
        """True when the step after `flight` is certain to be its requests again."""
        if not self.lookahead or self.scheduler.waiting or len(self.scheduler.running) != len(flight.entries):
            return False
        for e in flight.entries:
            r = e.request
            if r.cancelled or r.state != "running":
                return False
            if r.max_tokens is not None and len(r.output) + 1 >= r.max_tokens:
                return False  # the step in flight brings it to its limit
        return self.cache.free_pages() >= len(flight.entries)

    def sync(self) -> list[Request]:
        """Reads a step still in flight; returns the requests that ended in it."""
        flight, self._inflight = self._inflight, None
        return self._finish(flight) if flight is not None else []

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
