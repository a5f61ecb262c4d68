"""CUDA graphs for steps made of single decode tokens.

A decode step launches a few hundred small kernels; captured once per (number of
entries, block-table width), both rounded up to a few sizes, and replayed, the
host's part of a step is one buffer fill, one host-to-device copy and one graph
launch. Captures share one memory pool and the runner keeps a bounded number of
them, least recently used first out. The captured work is
the same Model.forward the eager step runs, followed by the sampling kernel;
only where its inputs live differs (fixed device buffers).
"""

from __future__ import annotations

import gc

import numpy as np
import torch

from ..kernels import ops
from ..models.model import HostStep, StepBatch

_ALIGN = 16


class _Layout:
    """Typed arrays packed into one byte buffer, each starting on 16 bytes."""

    def __init__(self, fields: list[tuple[str, np.dtype, tuple[int, ...]]]):
        self.fields = {}
        offset = 0
        for name, dtype, shape in fields:
            size = int(np.prod(shape)) * np.dtype(dtype).itemsize
            self.fields[name] = (offset, np.dtype(dtype), shape, size)
            offset += -(-size // _ALIGN) * _ALIGN
        self.nbytes = max(offset, _ALIGN)

    def host_views(self, buffer: np.ndarray) -> dict[str, np.ndarray]:
        return {name: buffer[o : o + size].view(dt).reshape(shape)
                for name, (o, dt, shape, size) in self.fields.items()}

    def device_views(self, buffer: torch.Tensor) -> dict[str, torch.Tensor]:
        kinds = {np.dtype(np.int32): torch.int32, np.dtype(np.float32): torch.float32,
                 np.dtype(np.int64): torch.int64}
        return {name: buffer[o : o + size].view(kinds[dt]).view(shape)
                for name, (o, dt, shape, size) in self.fields.items()}


class GraphedDecode:
    """One captured decode step for `n` entries and block tables `width` wide."""

    def __init__(self, runner, n: int, width: int, variants: dict | None = None):
        self.runner = runner
        self.n = n
        self.width = width
        self.variants = dict(variants or {})  # what the parts' plan_variant answered: see HostStep
        cache = runner.cache
        fields = [("tokens", np.int32, (n,)), ("source", np.int32, (n,)), ("pos", np.int32, (n,)),
                  ("entry", np.int32, (n,)),
                  ("slots", np.int32, (n,)), ("want", np.int32, (n,)), ("top_k", np.int32, (n,)),
                  ("temperature", np.float32, (n,)), ("top_p", np.float32, (n,)),
                  ("seed", np.int64, (n,)), ("count", np.int64, (n,))]
        fields += [(f"table{g.index}", np.int32, (n, width)) for g in cache.groups]
        # What the parts plan for a step of this shape: arrays get a place in the packed
        # buffer and are refreshed before every replay; the rest is kept as first planned.
        self.bound = width * cache.page_size
        first = self._host_step([self.bound] * n)
        self.plans: dict = {}
        self._planned_arrays: list[tuple] = []  # (part, key, name, field)
        for index, (key, part) in enumerate(runner._planners):
            plan = self.plans[key] = dict(part.plan_step(first))
            for name, value in plan.items():
                if isinstance(value, np.ndarray):
                    field = f"plan{index}.{name}"
                    fields.append((field, value.dtype, value.shape))
                    self._planned_arrays.append((part, key, name, field))
        self.layout = _Layout(fields)
        self.host = torch.empty(self.layout.nbytes, dtype=torch.uint8, pin_memory=True)
        self.h = self.layout.host_views(self.host.numpy())
        self.dev = torch.zeros(self.layout.nbytes, dtype=torch.uint8, device=runner.device)
        self.d = self.layout.device_views(self.dev)
        self.h["entry"][:] = np.arange(n, dtype=np.int32)
        self.h["want"][:] = np.arange(n, dtype=np.int32)
        for part, key, name, field in self._planned_arrays:
            self.plans[key][name] = self.d[field]
        self.batch = StepBatch(
            tokens=self.d["tokens"], pos=self.d["pos"], entry=self.d["entry"],
            tables={g.index: self.d[f"table{g.index}"] for g in cache.groups},
            slots=self.d["slots"], want_rows=self.d["want"], status=runner.status,
            n_tokens=n, n_entries=n, n_decode=n, host_query_lens=[1] * n, host_context_lens=[self.bound] * n,
            extras={"graph": True}, plans=self.plans,
        )
        self.logits: torch.Tensor | None = None
        self.ids: torch.Tensor | None = None
        self.graph: torch.cuda.CUDAGraph | None = None
        self.copied = torch.cuda.Event()
        self.launches = 0
        self._results: list[torch.Tensor] | None = None
        self._result_events: list[torch.cuda.Event] = []
        self._turn = 0

    def _host_step(self, context_lens: list[int]) -> HostStep:
        n = self.n
        lens = list(context_lens) + [1] * (n - len(context_lens))  # padding rows hold one token
        return HostStep(n_entries=n, n_tokens=n, n_decode=n, query_lens=[1] * n, context_lens=lens,
                        first_rows=list(range(n)), page_size=self.runner.cache.page_size, fixed_shape=True,
                        context_bound=self.bound, variants=self.variants)

    def pad_rows(self, n_real: int) -> None:
        """Rows past the step's `n_real` entries: token 0 at position 0 of each group's
        padding page, with the padding state slot, drawn greedily; nothing reads what they
        compute."""
        if n_real == self.n:
            return
        h = self.h
        for name in ("tokens", "pos", "top_k"):
            h[name][n_real:] = 0
        h["source"][n_real:] = -1
        h["slots"][n_real:] = self.runner.cache.pad_slot
        h["temperature"][n_real:] = 0.0
        h["top_p"][n_real:] = 2.0
        h["seed"][n_real:] = 0
        h["count"][n_real:] = 0
        for g in self.runner.cache.groups:
            table = h[f"table{g.index}"]
            table[n_real:] = -1
            table[n_real:, 0] = g.n_pages  # (the group's padding page)

    def plan(self, context_lens: list[int]) -> None:
        """Refreshes the arrays the parts planned, for this replay's lengths."""
        if not self._planned_arrays:
            return
        step = self._host_step(context_lens)
        fresh: dict = {}
        for part, key, name, field in self._planned_arrays:
            if key not in fresh:
                fresh[key] = part.plan_step(step)
            value = fresh[key][name]
            if value.shape != self.h[field].shape or value.dtype != self.h[field].dtype:
                raise ValueError(f"{type(part).__name__}.plan_step: array {name!r} changed from "
                                 f"{self.h[field].dtype}{self.h[field].shape} to {value.dtype}{value.shape} between "
                                 f"replays of one captured step; its shape may depend on the number of entries and "
                                 f"the context bound only")
            self.h[field][...] = value

    def _forward(self) -> None:
        self.logits = self.runner.model.forward(self.batch)
        # The sampled ids, and behind them the kernels' status word as it stands after
        # this step: both reach the host in the step's one copy.
        self._result = torch.empty(self.n + 1, dtype=torch.int32, device=self.runner.device)
        self.ids = self._result[: self.n]
        ops.sample(self.logits, self.d["temperature"], self.d["top_k"], self.d["top_p"], self.d["seed"],
                   self.d["count"], self.ids)
        self._result[self.n :].copy_(self.runner.status)

    def capture(self) -> None:
        """Runs the step once eagerly on a side stream (libraries set themselves up),
        then records it. The buffers must hold a valid batch."""
        self.dev.copy_(self.host, non_blocking=True)
        # The warm-up run really runs the step. Keys and values are written by position, so
        # running it twice changes nothing; the attention-mass accumulators are added to and
        # state slots are updated in place, so both are put back as they were.
        cache = self.runner.cache
        kept = [(g.mass_sum, g.mass_sum.clone(), g.weight_sum, g.weight_sum.clone())
                for g in cache.groups if g.mass_sum is not None]
        states = [(t, t.clone()) for t in cache.states.values()]  # (updated in place by their mixers)
        # One side stream for every capture of this runner: the allocator keeps freed blocks
        # per stream, so a new stream per capture would strand the warm-up's buffers.
        if self.runner._capture_stream is None:
            self.runner._capture_stream = torch.cuda.Stream()
        side = self.runner._capture_stream
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._forward()
        torch.cuda.current_stream().wait_stream(side)
        for mass, mass_before, weight, weight_before in kept:
            mass.copy_(mass_before)
            weight.copy_(weight_before)
        for state, before in states:
            state.copy_(before)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        # Nothing else may touch the device while the stream records: above all not the
        # collector, which could pick this moment to destroy another engine's graphs and
        # pools (calls that are not permitted during a capture and would invalidate it).
        gc.collect()
        collecting = gc.isenabled()
        gc.disable()
        try:
            if self.runner._graph_pool is None:
                self.runner._graph_pool = torch.cuda.graph_pool_handle()
            with torch.cuda.graph(self.graph, pool=self.runner._graph_pool, capture_error_mode="thread_local"):
                self._forward()
        finally:
            if collecting:
                gc.enable()
        self.launches = ops.launch_count() - before

    def replay(self, ids: torch.Tensor | None = None) -> None:
        """Copies the packed inputs and launches the graph. With `ids` (int32 on the device,
        the token ids an earlier step is drawing) the entries whose `source` row is not
        negative take their token from `ids[source]` instead of from the host buffer; the
        kernel that moves them is ordered after whatever writes `ids`."""
        self.dev.copy_(self.host, non_blocking=True)
        self.copied.record()
        if ids is not None:
            ops.take_tokens(self.d["tokens"], self.d["source"], ids, self.runner.status)
        self.graph.replay()

    def read_back(self) -> "PendingIds":
        """Starts the copy of this replay's sampled ids to the host; `wait()` on the result
        gives them. Two host buffers alternate, so one earlier result may still be unread."""
        if self._results is None:
            self._results = [torch.empty(self.n + 1, dtype=torch.int32, pin_memory=True) for _ in range(2)]
            self._result_events = [torch.cuda.Event(), torch.cuda.Event()]
        slot = self._turn
        self._turn ^= 1
        self._results[slot].copy_(self._result, non_blocking=True)
        self._result_events[slot].record()
        return PendingIds(self._results[slot], self._result_events[slot], self.runner)


class PendingIds:
    """Sampled token ids on their way to the host."""

    def __init__(self, host: torch.Tensor, event: torch.cuda.Event, runner):
        self._host = host
        self._event = event
        self._runner = runner

    def wait(self) -> list[int]:
        """The ids; raises if a kernel had flagged an error by the end of that step."""
        self._event.synchronize()  # the step's one synchronisation
        values = self._host.tolist()
        if values[-1]:
            self._runner.raise_status(values[-1])
        return values[:-1]
