"""The step function: one batch of (request, its next tokens) through the model.

A step runs only the tokens it is given, as one batch, against the cache that
earlier steps left: portions of prompts beside single decoded tokens, cut
anywhere. It reserves the pages the tokens need, uploads the batch's index
arrays in one copy, runs the model once over all tokens, and returns fp32
logits at the wanted places. The reference builds two groups per step and runs
the model over each (pulsarlm-core/src/engine/executor.cpp:187-268,
src/engine/model/paged_forward.cpp:136-145); here prompt portions and decode
tokens share one pass.
"""

from __future__ import annotations

import collections
import dataclasses

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..kernels import ops
from ..models.model import HostStep, Model, StepBatch


class OutOfPages(RuntimeError):
    """The cache has too few free pages (or slots) for a step's entry."""

    def __init__(self, request, message: str):
        super().__init__(message)
        self.request = request


@dataclasses.dataclass
class StepEntry:
    """`tokens`: the request's next tokens (at least one). `want`: indices into
    `tokens` whose logits the step returns, in this order."""

    request: object
    tokens: list[int]
    want: list[int] = dataclasses.field(default_factory=list)


STATUS_MESSAGES = {
    1: "a token id outside the vocabulary reached the embedding kernel",
    2: "a token's block-table entry was not a page of the pool when its key was written",
    4: "a block-table entry was not a page of the pool when attention read it",
    8: "a bounded wait inside a kernel gave up (a barrier or a copy that never arrived)",
}


def graph_entries_bucket(n: int) -> int:
    """How many entries the captured decode step that serves `n` entries has: n itself
    up to 4, then the next multiple of 4 up to 16, of 8 up to 64, of 16 beyond. The
    rows past n are padding (a token at position 0 of a page of their own that no
    request holds; their outputs are dropped), so a batch that shrinks as requests
    end passes through few captures."""
    if n <= 4:
        return n
    step = 4 if n <= 16 else 8 if n <= 64 else 16
    return -(-n // step) * step


def graph_width_bucket(pages: int) -> int:
    """Block-table width of the captured decode step that serves rows of `pages`
    pages: multiples of 64 up to 512, of 256 up to 2,048, of 1,024 beyond (at most an
    eighth more than needed from 512 pages on)."""
    step = 64 if pages <= 512 else 256 if pages <= 2048 else 1024
    return -(-pages // step) * step



class ModelRunner:
    def __init__(self, model: Model, cache: CacheManager):
        ops.require_device()
        self.model = model
        self.cache = cache
        self.device = model.ctx.device
        self.vocab = model.spec.vocab_size
        self._bindings = cache.bindings()
        self._bind()
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._staging: torch.Tensor | None = None
        self._planners = model.planners()
        self._variant_planners = [(key, part) for key, part in self._planners if hasattr(part, "plan_variant")]
        # Captured decode steps, least recently used first; at most `max_graphs` are kept
        # (each holds its own logits [entries, vocab] and small buffers; activations come
        # from one memory pool that all captures share).
        self._graphs: collections.OrderedDict = collections.OrderedDict()
        self.max_graphs = 24
        self._graph_pool = None
        self._capture_stream = None
        self.graph_captures = 0
        # Steps of single tokens are captured unless a part cannot take it. A mixer with state
        # slots must say that its single-token step can be captured (no host round trip in it):
        # `captures_state_steps()`; the capture's warm-up run then works on a copy of the states
        # and rows that pad a step use a slot no request holds. With attention mass measured,
        # steps are captured only if every mixer can measure inside one.
        state_mixers = [self.model.blocks[layer].mixer for layer in cache.state_layers]
        self.graphs_allowed = all(getattr(m, "captures_state_steps", lambda: False)() for m in state_mixers) and (
            cache.mass_decay is None or all(
                getattr(part, "measures_mass_in_captured_steps", lambda: True)() for part in model.parts()))
        self.steps = 0
        self.tokens_run = 0
        self.graph_steps = 0

    # ------------------------------------------------------------------ helpers
    def _bind(self) -> None:
        """Points the model's layers at this runner's cache. A model serves one cache at a
        time: when another runner was made over the same model since (a second engine
        sharing the weights), the layers are pointed back before this one steps."""
        if getattr(self.model, "bound_to", None) is not self:
            self.model.bind_caches(self._bindings)
            self.model.bound_to = self

    def _stage(self, arrays: list[np.ndarray]) -> list[torch.Tensor]:
        """Copies int32 arrays to the device through one pinned buffer and one copy;
        returns device views in the same order."""
        sizes = [a.size for a in arrays]
        # Views start on 16-byte boundaries (4 int32), which vector loads may rely on.
        starts, total = [], 0
        for s in sizes:
            starts.append(total)
            total += -(-s // 4) * 4
        total = max(total, 4)
        if self._staging is None or self._staging.numel() < total:
            self._staging = torch.empty(max(total, 4096), dtype=torch.int32, pin_memory=True)
        host = self._staging[:total]
        flat = host.numpy()
        for a, start in zip(arrays, starts):
            flat[start : start + a.size] = a.reshape(-1)
        dev = torch.empty(total, dtype=torch.int32, device=self.device)
        dev.copy_(host, non_blocking=True)
        # The pinned buffer is reused by the next step: the copy must have left it.
        if getattr(self, "_copy_done", None) is None:
            self._copy_done = torch.cuda.Event()
        self._copy_done.record()
        return [dev[start : start + a.size].view(a.shape) for a, start in zip(arrays, starts)]

    def prepare(self, entries: list[StepEntry], taken: tuple | None = None) -> tuple[StepBatch, list[int]]:
        """Reserves pages and builds the device batch; returns it with each entry's
        new length (to commit after the forward). taken: see `step`."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        sources = list(taken[1]) if taken is not None else [-1] * len(entries)
        if len(sources) != len(entries) or any(s >= 0 and len(e.tokens) != 1 for s, e in zip(sources, entries)):
            raise ValueError("tokens taken from the device: one row per entry, and only for entries of one token")
        seen = set()
        for e, source in zip(entries, sources):
            if e.request in seen:
                raise ValueError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.request!r}: a step entry needs at least one token")
            if n == 1:
                if source < 0 and not 0 <= int(e.tokens[0]) < self.vocab:
                    raise ValueError(f"request {e.request!r}: token id {e.tokens[0]} is outside [0, {self.vocab})")
            else:
                ids = np.asarray(e.tokens)
                if int(ids.min()) < 0 or int(ids.max()) >= self.vocab:
                    bad = [t for t in e.tokens if not 0 <= int(t) < self.vocab]
                    raise ValueError(f"request {e.request!r}: token id {bad[0]} is outside [0, {self.vocab})")
            if e.want and not all(0 <= w < n for w in e.want):
                raise ValueError(f"request {e.request!r}: wanted places {e.want} are outside its {n} tokens")
        for e in entries:
            if not self.cache.is_open(e.request):
                if self.cache.open(e.request) is None:
                    raise OutOfPages(e.request, f"no free slot for request {e.request!r}")
        all_requests = [e.request for e in entries]
        starts, all_slots, done = self.cache.reserve_many(all_requests, [len(e.tokens) for e in entries])
        if done < len(entries):
            e = entries[done]
            raise OutOfPages(e.request, f"too few free pages for request {e.request!r} to reach "
                                        f"{int(starts[done]) + len(e.tokens)} tokens")
        new_lens = [int(starts[i]) + len(e.tokens) for i, e in enumerate(entries)]

        if getattr(self, "_copy_done", None) is not None:
            self._copy_done.synchronize()
        # Entries of one token go first (StepBatch's contract: mixers may send the leading
        # single tokens to a kernel of their own); the wanted rows still come back in the
        # caller's order of entries.
        order = sorted(range(len(entries)), key=lambda i: len(entries[i].tokens) != 1)
        n_decode = sum(1 for e in entries if len(e.tokens) == 1)
        n_tokens = sum(len(e.tokens) for e in entries)
        tokens = np.empty(n_tokens, dtype=np.int32)
        pos = np.empty(n_tokens, dtype=np.int32)
        entry = np.empty(n_tokens, dtype=np.int32)
        first_row = [0] * len(entries)
        at = 0
        for place, i in enumerate(order):
            e = entries[i]
            n = len(e.tokens)
            start = int(starts[i])
            tokens[at : at + n] = e.tokens if sources[i] < 0 else 0
            if n == 1:
                pos[at] = start
            else:
                pos[at : at + n] = np.arange(start, start + n, dtype=np.int32)
            entry[at : at + n] = place
            first_row[i] = at
            at += n
        want_rows = [first_row[i] + w for i, e in enumerate(entries) for w in e.want]
        requests = [entries[i].request for i in order]
        slots = all_slots[order]
        tables = [self.cache.table_rows(g.index, requests) for g in self.cache.groups]
        host = HostStep(n_entries=len(entries), n_tokens=n_tokens, n_decode=n_decode,
                        query_lens=[len(entries[i].tokens) for i in order],
                        context_lens=[new_lens[i] for i in order],
                        first_rows=[first_row[i] for i in order], page_size=self.cache.page_size)
        arrays = [tokens, pos, entry, slots, np.array(want_rows, dtype=np.int32), *tables]
        n_fixed = len(arrays)
        # What the parts plan for this step: their arrays travel in the same copy.
        plans: dict = {}
        staged: list[tuple] = []  # (plan key, name, index into arrays, is float)
        for key, part in self._planners:
            plan = plans[key] = dict(part.plan_step(host))
            for name, value in plan.items():
                if isinstance(value, np.ndarray):
                    if value.dtype not in (np.int32, np.float32):
                        raise TypeError(f"{type(part).__name__}.plan_step: array {name!r} must be int32 or float32, "
                                        f"not {value.dtype}")
                    staged.append((key, name, len(arrays), value.dtype == np.float32))
                    arrays.append(np.ascontiguousarray(value).view(np.int32))
        decay = self.cache.mass_decay
        n_planned = len(arrays)
        if decay is not None:
            # Query weights a (1 - a)^age within each portion, and per page what the
            # accumulators keep: (1 - a)^tokens for pages the step's requests held, 0
            # for pages taken for this step (they may hold a former owner's sums).
            weights = np.empty(n_tokens, dtype=np.float32)
            at = 0
            for i in order:
                n = len(entries[i].tokens)
                weights[at : at + n] = decay * (1.0 - decay) ** np.arange(n - 1, -1, -1, dtype=np.float64)
                at += n
            arrays.append(weights.view(np.int32))
            for g in self.cache.groups:
                keep = np.ones(g.n_pages + 1, dtype=np.float32)
                for e in entries:
                    keep[self.cache.held_pages(e.request, g.index)] = (1.0 - decay) ** len(e.tokens)
                keep[list(self.cache.take_fresh_pages(g.index))] = 0.0
                arrays.append(keep.view(np.int32))
        if taken is not None and n_decode and max(sources) >= 0:
            # (entries of one token lead the batch: their rows are the first n_decode)
            arrays.append(np.array([sources[i] for i in order[:n_decode]], dtype=np.int32))
        else:
            taken = None
        dev = self._stage(arrays)
        if taken is not None:
            ops.take_tokens(dev[0], dev[-1], taken[0], self.status)
        for key, name, index, is_float in staged:
            plans[key][name] = dev[index].view(torch.float32) if is_float else dev[index]
        batch = StepBatch(
            tokens=dev[0], pos=dev[1], entry=dev[2],
            tables={g.index: dev[5 + i] for i, g in enumerate(self.cache.groups)},
            slots=dev[3],
            want_rows=dev[4] if want_rows else None,
            status=self.status,
            n_tokens=n_tokens,
            n_entries=len(entries),
            n_decode=n_decode,
            host_query_lens=host.query_lens,
            host_context_lens=host.context_lens,
            plans=plans,
        )
        assert n_fixed == 5 + len(self.cache.groups)
        if decay is not None:
            batch.extras["query_weights"] = dev[n_planned].view(torch.float32)
            batch.extras["mass_retained"] = {g.index: dev[n_planned + 1 + i].view(torch.float32)
                                             for i, g in enumerate(self.cache.groups)}
        return batch, new_lens

    # ------------------------------------------------------------------ the step
    def step(self, entries: list[StepEntry], taken: tuple | None = None) -> torch.Tensor | None:
        """Runs the entries' tokens; returns fp32 logits [wanted, vocab] on the device
        in the order of the entries and of each entry's `want`, or None. taken: (ids,
        rows) with `ids` an int32 device tensor (the token ids an earlier step is still
        drawing) and `rows[i]` the row of `ids` that holds entry i's one token, or -1 for
        an entry whose tokens are its own."""
        self._bind()
        batch, new_lens = self.prepare(entries, taken)
        logits = self.model.forward(batch)
        if self.cache.mass_decay is not None:
            self.cache.fold_mass(batch.extras["mass_retained"])
        self.cache.commit_many([e.request for e in entries], new_lens)
        self.steps += 1
        self.tokens_run += batch.n_tokens
        return logits

    def decode_step(self, entries: list[StepEntry], sampling, seeds: list[int], counts: list[int],
                    taken: tuple | None = None) -> torch.Tensor:
        """A step of single tokens, one per entry, each sampling its next token:
        replays a CUDA graph captured for this number of entries (rounded up, see
        graph_entries_bucket). Returns int32 token ids, the entries' first, in a device
        buffer that the next call overwrites
        (`self.last_graph.read_back()` starts their copy to the host). taken: as in
        `step` (tokens that a step still under way is drawing)."""
        from .graphs import GraphedDecode

        self._bind()  # (a replay runs on the pools it was captured with; a capture needs the binding)
        n = len(entries)
        new_lens = []
        for e in entries:
            if len(e.tokens) != 1:
                raise ValueError("decode_step takes entries of one token")
            if not self.cache.is_open(e.request):
                raise ValueError(f"request {e.request!r} has no cache to decode from")
            new_len = self.cache.length(e.request) + 1
            if not self.cache.reserve(e.request, new_len):
                raise OutOfPages(e.request, f"too few free pages for request {e.request!r} to reach {new_len} tokens")
            new_lens.append(new_len)
        pages = -(-max(new_lens) // self.cache.page_size)
        width = graph_width_bucket(pages)
        n_graph = graph_entries_bucket(n)
        # Parts may want a capture of their own for some replays (see HostStep.variants).
        variants = {}
        if self._variant_planners:
            host = HostStep(n_entries=n, n_tokens=n, n_decode=n, query_lens=[1] * n, context_lens=new_lens,
                            first_rows=list(range(n)), page_size=self.cache.page_size, fixed_shape=True,
                            context_bound=width * self.cache.page_size)
            variants = {key: part.plan_variant(host) for key, part in self._variant_planners}
        key = (n_graph, width, *sorted((repr(k), repr(v)) for k, v in variants.items() if v is not None))
        graph = self._graphs.get(key)
        fresh = graph is None
        if fresh:
            graph = GraphedDecode(self, n_graph, width, variants)
            self._graphs[key] = graph
            while len(self._graphs) > max(2, self.max_graphs):
                # The least recently used capture goes; its buffers return to the shared
                # pool once nothing in flight holds them (the two most recent never go).
                self._graphs.popitem(last=False)
        else:
            self._graphs.move_to_end(key)
            graph.copied.synchronize()
        h = graph.h
        requests = [e.request for e in entries]
        for i, e in enumerate(entries):
            source = taken[1][i] if taken is not None else -1
            h["tokens"][i] = e.tokens[0] if source < 0 else 0
            h["source"][i] = source
            h["pos"][i] = new_lens[i] - 1
            p = sampling[i]
            h["temperature"][i] = p.temperature if p.draws else 0.0
            h["top_k"][i] = p.top_k
            h["top_p"][i] = p.top_p if 0.0 < p.top_p < 1.0 else 2.0
            h["seed"][i] = np.uint64(seeds[i] & 0xFFFFFFFFFFFFFFFF).astype(np.int64)
            h["count"][i] = counts[i]
        handles = [self.cache.handle(r) for r in requests]
        for g in self.cache.groups:
            table = h[f"table{g.index}"]
            self.cache.fill_tables(g.index, handles, table[:n], h["slots"][:n])
        if self.cache.mass_decay is not None:
            # The kernels see which page a token opens; the host's list of pages taken since
            # the last eager step is not needed and must not reach that step.
            for g in self.cache.groups:
                self.cache.take_fresh_pages(g.index)
        graph.pad_rows(n)
        graph.plan(new_lens)
        if fresh:
            graph.capture()
            self.graph_captures += 1
        graph.replay(taken[0] if taken is not None and max(taken[1]) >= 0 else None)
        self.last_graph = graph
        for e, new_len in zip(entries, new_lens):
            self.cache.commit(e.request, new_len)
        self.steps += 1
        self.graph_steps += 1
        self.tokens_run += n
        return graph.ids

    def end(self, request) -> None:
        """Gives back what the request holds."""
        if self.cache.is_open(request):
            self.cache.close(request)

    def check_status(self) -> None:
        """Raises if a kernel flagged an error since the last check (synchronises)."""
        code = int(self.status.item())
        if code:
            self.raise_status(code)

    def raise_status(self, code: int) -> None:
        """Clears the device status word and raises what `code` (a copy of it) says."""
        self.status.zero_()
        reasons = [m for bit, m in STATUS_MESSAGES.items() if code & bit]
        raise RuntimeError("kernel status %d: %s" % (code, "; ".join(reasons) or "unknown"))
