"""The cache manager: paged keys and values per layer group, block tables per
request, and fixed-size state slots.

Layers whose mixers ask for the same KVCacheNeed (kv heads, head size, window)
form a group. A group has its own page pool: one tensor
[layers in group, pages, 2 (K, V), kv heads, page size, head size], so one page
id holds `page_size` tokens of every layer of the group, and a request has one
block table per group. Groups with a window give pages back as soon as every
token in them is out of every future query's reach. Mixers that ask for a
StateNeed get a row per request slot in a tensor [slots, *shape], zeroed when
the slot is handed out.

A request's life: `open` (a slot) -> `reserve(new_len)` before each step (pages
for the step's tokens, all groups or none) -> `commit(new_len)` after it (length
recorded, passed window pages given back) -> `close` (everything given back).

The reference keeps one byte pool cut into per-layer "lines"
(pulsarlm-core/src/engine/kv_cache.cpp:96-164, 310-423), releases lines at
finish (src/engine/executor.cpp:695-700) and pages that slid out of a window
during the run (executor.cpp:702-715); its recurrent layers hold fixed lines
(src/engine/sequence.cpp:361-362).
"""

from __future__ import annotations

import dataclasses

import numpy as np
import torch

from ..parts.attention import KVBinding
from ..parts.spec import KVCacheNeed, StateNeed
from .pages import PagePool


class CacheError(RuntimeError):
    pass


@dataclasses.dataclass
class StateBinding:
    """What a mixer that asked for a StateNeed gets: `states[slot]` is the state
    of the request in that slot; `batch.slots` names each entry's slot."""

    states: torch.Tensor


@dataclasses.dataclass
class _Group:
    index: int
    need: KVCacheNeed
    layers: list[int]
    pool: PagePool
    tensor: torch.Tensor | None
    # attention mass, when measured: accumulators and this step's sums
    mass_sum: torch.Tensor | None = None     # [layers, pages, query heads]
    weight_sum: torch.Tensor | None = None   # [layers, pages]
    step_mass: torch.Tensor | None = None
    step_weight: torch.Tensor | None = None


@dataclasses.dataclass
class _Request:
    slot: int
    length: int = 0
    # Per group: page id of every page index so far, -1 once given back.
    pages: list[list[int]] = dataclasses.field(default_factory=list)


_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


class CacheManager:
    def __init__(self, needs: list, page_size: int, n_pages: int, max_requests: int, dtype: torch.dtype,
                 device: torch.device | str | None, allocate: bool = True, mass_decay: float | None = None):
        """needs: per layer KVCacheNeed, StateNeed or None. n_pages: pages of every
        group's pool. allocate=False keeps the bookkeeping only (no tensors).
        mass_decay: when given (0 < a <= 1), per-page attention-mass accumulators are
        kept: each step the attention kernel adds, for every page a query attends,
        w * (the query's largest scaled score in the page) per head and w per page,
        with w = a (1 - a)^age for the query `age` tokens before the end of its
        portion; before a step's sums are added, what a request's pages hold is
        scaled by (1 - a)^(tokens in the step)
        (pulsarlm-core/src/engine/eviction.cpp:115-138). Nothing is evicted."""
        if page_size <= 0 or n_pages <= 0 or max_requests <= 0:
            raise ValueError("page_size, n_pages and max_requests must be positive")
        if mass_decay is not None and not 0.0 < mass_decay <= 1.0:
            raise ValueError("mass_decay must be in (0, 1]")
        self.mass_decay = mass_decay
        self.page_size = page_size
        self.n_pages = n_pages
        self.max_requests = max_requests
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else None
        self.groups: list[_Group] = []
        self.layer_group: dict[int, int] = {}
        self.state_layers: dict[int, StateNeed] = {}
        self.states: dict[int, torch.Tensor] = {}
        by_need: dict[KVCacheNeed, _Group] = {}
        for layer, need in enumerate(needs):
            if isinstance(need, KVCacheNeed):
                group = by_need.get(need)
                if group is None:
                    group = _Group(len(self.groups), need, [], PagePool(n_pages), None)
                    by_need[need] = group
                    self.groups.append(group)
                self.layer_group[layer] = group.index
                group.layers.append(layer)
            elif isinstance(need, StateNeed):
                self.state_layers[layer] = need
            elif need is not None:
                raise ValueError(f"layer {layer}: unknown cache need {need!r}")
        if allocate:
            for group in self.groups:
                n = group.need
                group.tensor = torch.zeros(
                    (len(group.layers), n_pages, 2, n.n_kv_heads, page_size, n.head_dim), dtype=dtype, device=device)
            if mass_decay is not None:
                for group in self.groups:
                    shape = (len(group.layers), n_pages, max(1, group.need.n_heads))
                    group.mass_sum = torch.zeros(shape, dtype=torch.float32, device=device)
                    group.step_mass = torch.zeros(shape, dtype=torch.float32, device=device)
                    group.weight_sum = torch.zeros(shape[:2], dtype=torch.float32, device=device)
                    group.step_weight = torch.zeros(shape[:2], dtype=torch.float32, device=device)
            for layer, need in self.state_layers.items():
                self.states[layer] = torch.zeros((max_requests, *need.shape), dtype=_STATE_DTYPES[need.dtype],
                                                 device=device)
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self._requests: dict[object, _Request] = {}
        # Pages taken since the last step (their mass accumulators must restart at zero).
        self._fresh: list[set] = [set() for _ in self.groups]

    # ------------------------------------------------------------------ bindings
    def bindings(self) -> list:
        """Per layer: KVBinding, StateBinding or None, for `Model.bind_caches`."""
        n_layers = max([*self.layer_group, *self.state_layers, -1]) + 1
        out: list = [None] * n_layers
        for layer, g in self.layer_group.items():
            group = self.groups[g]
            where = group.layers.index(layer)
            out[layer] = KVBinding(g, group.tensor[where, :, 0], group.tensor[where, :, 1], self.page_size,
                                   group.step_mass[where] if group.step_mass is not None else None,
                                   group.step_weight[where] if group.step_weight is not None else None)
        for layer in self.state_layers:
            out[layer] = StateBinding(self.states[layer])
        return out

    def bytes_per_page(self) -> int:
        width = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.layers) * 2 * g.need.n_kv_heads * self.page_size * g.need.head_dim * width
                   for g in self.groups)

    # ------------------------------------------------------------------ requests
    def open(self, request) -> int | None:
        """A slot for a new request (its states zeroed), or None when all are taken."""
        if request in self._requests:
            raise CacheError(f"request {request!r} is already open")
        if not self._free_slots:
            return None
        slot = self._free_slots.pop()
        self._requests[request] = _Request(slot, 0, [[] for _ in self.groups])
        for states in self.states.values():
            states[slot].zero_()
        return slot

    def is_open(self, request) -> bool:
        return request in self._requests

    def slot(self, request) -> int:
        return self._requests[request].slot

    def length(self, request) -> int:
        return self._requests[request].length

    def _first_needed_page(self, group: _Group, length: int) -> int:
        """Index of the first page a query at position >= `length` can still read."""
        if group.need.window is None:
            return 0
        first_key = max(0, length - group.need.window + 1)
        return first_key // self.page_size

    def pages_needed(self, request, new_len: int) -> int:
        """Pages `reserve(request, new_len)` would take, summed over groups."""
        r = self._requests[request]
        n_pages = -(-new_len // self.page_size)
        return sum(max(0, n_pages - len(r.pages[g.index])) for g in self.groups)

    def reserve(self, request, new_len: int) -> bool:
        """Pages so that tokens [0, new_len) have a place in every group. Takes all
        that is missing or nothing; False when some pool has too few free pages."""
        r = self._requests[request]
        if new_len < r.length:
            raise CacheError(f"request {request!r} cannot shrink from {r.length} to {new_len} tokens")
        n_pages = -(-new_len // self.page_size)
        missing = [max(0, n_pages - len(r.pages[g.index])) for g in self.groups]
        if any(m > g.pool.free_count for m, g in zip(missing, self.groups)):
            return False
        for m, g in zip(missing, self.groups):
            taken = g.pool.take(m)
            r.pages[g.index].extend(taken)
            if self.mass_decay is not None:
                self._fresh[g.index].update(taken)
        return True

    def commit(self, request, new_len: int) -> None:
        """Records that tokens [0, new_len) are cached; gives back the pages of
        windowed groups that no later query can reach."""
        r = self._requests[request]
        if new_len < r.length or any(-(-new_len // self.page_size) > len(p) for p in r.pages):
            raise CacheError(f"request {request!r}: commit({new_len}) without pages reserved")
        r.length = new_len
        for g in self.groups:
            pages = r.pages[g.index]
            first = self._first_needed_page(g, new_len)
            passed = [i for i in range(min(first, len(pages))) if pages[i] >= 0]
            if passed:
                g.pool.give([pages[i] for i in passed])
                for i in passed:
                    pages[i] = -1

    def close(self, request) -> None:
        """Gives back every page and the slot of the request."""
        r = self._requests.pop(request)
        for g in self.groups:
            g.pool.give([p for p in r.pages[g.index] if p >= 0])
        self._free_slots.append(r.slot)

    def open_requests(self) -> list:
        return list(self._requests)

    # ------------------------------------------------------------------ tables
    def table_rows(self, group: int, requests: list, width_multiple: int = 8) -> np.ndarray:
        """int32 [len(requests), W]: each request's page ids of `group`, -1 where it
        holds none; W is the longest row rounded up to `width_multiple`."""
        rows = [self._requests[r].pages[group] for r in requests]
        width = max([len(row) for row in rows] + [1])
        width = -(-width // width_multiple) * width_multiple
        table = np.full((len(rows), width), -1, dtype=np.int32)
        for i, row in enumerate(rows):
            table[i, : len(row)] = row
        return table

    def held_pages(self, request, group: int) -> list[int]:
        return [p for p in self._requests[request].pages[group] if p >= 0]

    # ------------------------------------------------------------------ attention mass
    def take_fresh_pages(self, group: int) -> set:
        """Pages of `group` taken since the last call: their accumulators hold a former
        owner's sums until the next fold clears them."""
        fresh, self._fresh[group] = self._fresh[group], set()
        return fresh

    def fold_mass(self, retained: dict[int, torch.Tensor]) -> None:
        """After a step: accumulators = accumulators * retained[page] + the step's sums;
        the step's sums are cleared. retained[g]: fp32 [pages] on the device (1 for
        pages no entry of the step owns, 0 for pages taken in this step)."""
        for group in self.groups:
            if group.mass_sum is None:
                continue
            keep = retained[group.index]
            group.mass_sum.mul_(keep[None, :, None]).add_(group.step_mass)
            group.weight_sum.mul_(keep[None, :]).add_(group.step_weight)
            group.step_mass.zero_()
            group.step_weight.zero_()

    def page_mass(self, request, group: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
        """(mass_sum [layers, pages of the request, heads], weight_sum [layers, pages])
        of the pages the request holds in `group`, in the request's page order."""
        g = self.groups[group]
        if g.mass_sum is None:
            raise CacheError("attention mass is not being measured (mass_decay was not given)")
        pages = torch.tensor(self.held_pages(request, group), dtype=torch.long, device=g.mass_sum.device)
        return g.mass_sum[:, pages], g.weight_sum[:, pages]

    # ------------------------------------------------------------------ figures
    def stats(self) -> dict:
        return {
            "page_size": self.page_size,
            "groups": [
                {"layers": len(g.layers), "window": g.need.window, "pages": g.pool.n_pages,
                 "used": g.pool.used_count, "free": g.pool.free_count, "high_water": g.pool.high_water}
                for g in self.groups
            ],
            "slots": self.max_requests,
            "slots_used": self.max_requests - len(self._free_slots),
        }

    def free_pages(self) -> int:
        """Free pages of the fullest pool (what limits the next reservation)."""
        return min((g.pool.free_count for g in self.groups), default=self.n_pages)
