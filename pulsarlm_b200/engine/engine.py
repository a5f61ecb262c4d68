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
from typing import Iterator

import torch

from ..cache.manager import CacheManager
from ..kernels import ops
from ..models.model import Model
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .loading import load_model, parse_dtype, random_model
from .runner import ModelRunner, StepEntry
from .scheduler import PlannedEntry, Request, Scheduler

DEFAULT_PAGE_SIZE = 16


class Engine:
    def __init__(self, model, dtype="bfloat16", device="cuda:0", kv_cache_gib: float = 4.0,
                 page_size: int = DEFAULT_PAGE_SIZE, prefill_tokens_per_step: int = 256,
                 max_requests: int = 64, n_pages: int | None = None, stop_ids=None, seed: int | None = None,
                 cuda_graphs: bool = True, attention_mass_decay: float | None = None):
        """model: a model folder, a built Model, or a config.json dict (random
        weights from `seed`). kv_cache_gib sizes the page pools unless n_pages
        gives the number of pages outright. stop_ids default to config.json's
        eos_token_id. attention_mass_decay: measure per-page attention mass with this
        decay (see CacheManager; slower: attention then runs on the CUDA cores)."""
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
        if n_pages is None:
            probe = CacheManager(needs, page_size, 1, 1, self.dtype, None, allocate=False)
            per_page = max(1, probe.bytes_per_page())
            n_pages = max(1, int(kv_cache_gib * (1 << 30)) // per_page)
        self.cache = CacheManager(needs, page_size, n_pages, max_requests, self.dtype, self.device,
                                  mass_decay=attention_mass_decay)
        self.runner = ModelRunner(self.model, self.cache)
        self.sampler = Sampler(self.device)
        stops = self.model.spec.eos_token_ids if stop_ids is None else stop_ids
        self.scheduler = Scheduler(self.cache, stops, prefill_tokens_per_step)
        self.cuda_graphs = cuda_graphs and self.runner.graphs_allowed
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
        return self.scheduler.has_work()

    def step(self) -> list[Request]:
        """Runs one scheduler step on the GPU; returns the requests that ended in it."""
        entries, ended = self.scheduler.plan()
        if not entries:
            return ended
        step_entries = [StepEntry(e.request.id, e.tokens, [len(e.tokens) - 1] if e.samples else [])
                        for e in entries]
        sampled: dict = {}
        samplers = [e for e in entries if e.samples]
        if self.cuda_graphs and all(len(e.tokens) == 1 and e.samples and e.request.max_tokens != 0
                                    for e in entries):
            drawn = self.runner.decode_step(
                step_entries, [e.request.sampling for e in entries], [e.request.seed for e in entries],
                [e.request.draw_count for e in entries])
            host = drawn.cpu().tolist()  # the step's one synchronisation
            sampled = {e.request.id: t for e, t in zip(entries, host)}
            return ended + self.scheduler.finish_step(entries, sampled)
        logits = self.runner.step(step_entries)
        if samplers and logits is not None:
            drawn = self.sampler.sample(
                logits, [e.request.sampling for e in samplers], [e.request.seed for e in samplers],
                [e.request.draw_count for e in samplers])
            host = drawn.cpu().tolist()  # the step's one synchronisation
            sampled = {e.request.id: t for e, t in zip(samplers, host)}
        return ended + self.scheduler.finish_step(entries, sampled)

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
