"""The cache manager: paged keys and values per layer group, block tables per
request, and fixed-size state slots.

Layers whose mixers ask for the same KVCacheNeed (kv heads, head size, window)
form a group. A group has its own page pool: one tensor
[layers in group, pages + 1, 2 (K, V), kv heads, page size, head size] (the last
page is never handed out: padding rows of captured steps use it), so one page
id holds `page_size` tokens of every layer of the group, and a request has one
block table per group. Groups with a window give pages back as soon as every
token in them is out of every future query's reach, and when the caller bounds
the tokens a request brings to one step their pools are made only as large as
`max_requests` such requests can fill (`window_pages`). Mixers that ask for a
StateNeed get a row per request slot in a tensor [slots, *shape], zeroed when
the slot is handed out.

A request's life: `open` (a slot) -> `reserve(new_len)` before each step (pages
for the step's tokens, all groups or none) -> `commit(new_len)` after it (length
recorded, passed window pages given back) -> `close` (everything given back).

The bookkeeping (pools, slots, page lists) is C++: class CacheBook in
pulsarlm_b200/csrc_host/host_core.cpp. This class owns the tensors, groups the
layers, and maps the caller's request keys to the book's integer handles.

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

import ctypes

from ..host import core
from ..parts.attention import KVBinding
from ..parts.spec import KVCacheNeed, StateNeed
from .pages import GroupPoolView, PageError


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
    pool: GroupPoolView | None
    tensor: torch.Tensor | None
    n_pages: int = 0    # pages the pool hands out; page `n_pages` of the tensor is the padding page
    # attention mass, when measured: accumulators and this step's sums
    mass_sum: torch.Tensor | None = None     # [layers, pages, query heads]
    weight_sum: torch.Tensor | None = None   # [layers, pages]
    step_mass: torch.Tensor | None = None
    step_weight: torch.Tensor | None = None


_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


def window_pages(window: int, page_size: int, step_tokens: int, max_requests: int) -> int:
    """Pages that `max_requests` requests can hold at once in a group whose queries
    reach `window` keys back, when no request brings more than `step_tokens` tokens to
    a step. A request of length L that reserves n more tokens holds the pages from
    that of key L - window + 1 to that of key L + n - 1: fewer than
    (window + n - 1) / page_size + 2. One token more, for a step that is reserved
    while the step before it has not been committed."""
    per_request = -(-(window + step_tokens + 1) // page_size) + 1
    return max_requests * per_request


def pool_pages(need: KVCacheNeed, n_pages: int, page_size: int, step_tokens: int | None, max_requests: int) -> int:
    """Pages of the pool of a group with this need, when groups that keep every key get n_pages."""
    if need.window is None or step_tokens is None:
        return n_pages
    return min(n_pages, window_pages(need.window, page_size, step_tokens, max_requests))


def cache_bytes(needs: list, n_pages: int, page_size: int, step_tokens: int | None, max_requests: int,
                dtype: torch.dtype) -> int:
    """Bytes of the page tensors `CacheManager(needs, page_size, n_pages, ...)` would make
    (without the padding pages)."""
    width = torch.empty((), dtype=dtype).element_size()
    layers: dict[KVCacheNeed, int] = {}
    for need in needs:
        if isinstance(need, KVCacheNeed):
            layers[need] = layers.get(need, 0) + 1
    return sum(pool_pages(need, n_pages, page_size, step_tokens, max_requests)
               * count * 2 * need.n_kv_heads * page_size * need.head_dim * width for need, count in layers.items())


class CacheManager:
    def __init__(self, needs: list, page_size: int, n_pages: int, max_requests: int, dtype: torch.dtype,
                 device: torch.device | str | None, allocate: bool = True, mass_decay: float | None = None,
                 step_tokens: int | None = None):
        """needs: per layer KVCacheNeed, StateNeed or None. n_pages: pages of the pool
        of a group that keeps every key. step_tokens: the most tokens one request
        brings to a step, if the caller keeps to such a bound (a scheduler's token
        budget); a group with a window then gets `window_pages(...)` pages when that
        is fewer. Without it every group gets n_pages.
        allocate=False keeps the bookkeeping only (no tensors).
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
        # Likewise one more state slot than requests: the rows that pad a captured step update it.
        self.pad_slot = max_requests
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else None
        self.n_layers = len(needs)
        self.groups: list[_Group] = []
        self.layer_group: dict[int, int] = {}
        self.state_layers: dict[int, StateNeed] = {}
        self.states: dict[int, torch.Tensor] = {}
        by_need: dict[KVCacheNeed, _Group] = {}
        for layer, need in enumerate(needs):
            if isinstance(need, KVCacheNeed):
                group = by_need.get(need)
                if group is None:
                    group = _Group(len(self.groups), need, [], None, None)
                    by_need[need] = group
                    self.groups.append(group)
                self.layer_group[layer] = group.index
                group.layers.append(layer)
            elif isinstance(need, StateNeed):
                self.state_layers[layer] = need
            elif need is not None:
                raise ValueError(f"layer {layer}: unknown cache need {need!r}")
        for group in self.groups:
            group.n_pages = pool_pages(group.need, n_pages, page_size, step_tokens, max_requests)
        if allocate:
            # One more page than a pool hands out: the padding page (`group.n_pages`), which no
            # request ever holds. Rows that pad a captured decode step to its size write and read there.
            for group in self.groups:
                n = group.need
                group.tensor = torch.zeros(
                    (len(group.layers), group.n_pages + 1, 2, n.n_kv_heads, page_size, n.head_dim), dtype=dtype,
                    device=device)
            if mass_decay is not None:
                for group in self.groups:
                    shape = (len(group.layers), group.n_pages + 1, max(1, group.need.n_heads))
                    group.mass_sum = torch.zeros(shape, dtype=torch.float32, device=device)
                    group.step_mass = torch.zeros(shape, dtype=torch.float32, device=device)
                    group.weight_sum = torch.zeros(shape[:2], dtype=torch.float32, device=device)
                    group.step_weight = torch.zeros(shape[:2], dtype=torch.float32, device=device)
            for layer, need in self.state_layers.items():
                self.states[layer] = torch.zeros((max_requests + 1, *need.shape), dtype=_STATE_DTYPES[need.dtype],
                                                 device=device)
        self._lib = core.library()
        windows = (ctypes.c_int32 * max(1, len(self.groups)))(
            *[g.need.window if g.need.window is not None else -1 for g in self.groups])
        pages = (ctypes.c_int32 * max(1, len(self.groups)))(*[g.n_pages for g in self.groups])
        self._book = self._lib.plh_cache_create(len(self.groups), windows, page_size, pages, max_requests,
                                                int(mass_decay is not None))
        for group in self.groups:
            group.pool = GroupPoolView(self._lib, self._book, group.index, group.n_pages)
        # The caller's request keys (any hashable) <-> the book's integer handles.
        self._handles: dict[object, int] = {}
        self._keys: dict[int, object] = {}
        self._next_handle = 1
        self._row = (ctypes.c_int32 * max(1, n_pages))()

    def __del__(self):
        if getattr(self, "_book", None):
            self._lib.plh_cache_destroy(self._book)
            self._book = None

    # ------------------------------------------------------------------ handles
    @property
    def book(self):
        """The C++ CacheBook (for the scheduler core, which works on the same book)."""
        return self._book

    def handle(self, request) -> int:
        """The integer the book knows `request` by (made on first use)."""
        h = self._handles.get(request)
        if h is None:
            h = self._handles[request] = self._next_handle
            self._keys[h] = request
            self._next_handle += 1
        return h

    def key_of(self, handle: int):
        return self._keys[handle]

    def forget(self, request) -> None:
        """Drops the key <-> handle entry of a request that is closed for good."""
        h = self._handles.pop(request, None)
        if h is not None:
            self._keys.pop(h, None)

    def _known(self, request) -> int:
        h = self._handles.get(request)
        if h is None or not self._lib.plh_cache_is_open(self._book, h):
            raise KeyError(request)
        return h

    def zero_states(self, slot: int) -> None:
        for states in self.states.values():
            states[slot].zero_()

    # ------------------------------------------------------------------ bindings
    def bindings(self) -> list:
        """Per layer: KVBinding, StateBinding or None, for `Model.bind_caches`."""
        n_layers = self.n_layers
        out: list = [None] * n_layers
        for layer, g in self.layer_group.items():
            group = self.groups[g]
            where = group.layers.index(layer)
            out[layer] = KVBinding(g, group.tensor[where, :, 0], group.tensor[where, :, 1], self.page_size,
                                   group.step_mass[where] if group.step_mass is not None else None,
                                   group.step_weight[where] if group.step_weight is not None else None,
                                   group.mass_sum[where] if group.mass_sum is not None else None,
                                   group.weight_sum[where] if group.weight_sum is not None else None,
                                   self.mass_decay)
        for layer in self.state_layers:
            out[layer] = StateBinding(self.states[layer])
        return out

    def bytes_per_page(self) -> int:
        """Bytes of one page id in every group (a token count's worth of every layer)."""
        return sum(self.group_bytes_per_page(g.index) for g in self.groups)

    def group_bytes_per_page(self, group: int) -> int:
        g = self.groups[group]
        width = torch.empty((), dtype=self.dtype).element_size()
        return len(g.layers) * 2 * g.need.n_kv_heads * self.page_size * g.need.head_dim * width

    # ------------------------------------------------------------------ requests
    def open(self, request) -> int | None:
        """A slot for a new request (its states zeroed), or None when all are taken."""
        slot = self._lib.plh_cache_open(self._book, self.handle(request))
        if slot == core.ALREADY_OPEN:
            raise CacheError(f"request {request!r} is already open")
        if slot < 0:
            return None
        self.zero_states(slot)
        return slot

    def is_open(self, request) -> bool:
        h = self._handles.get(request)
        return h is not None and bool(self._lib.plh_cache_is_open(self._book, h))

    def slot(self, request) -> int:
        return self._lib.plh_cache_slot(self._book, self._known(request))

    def length(self, request) -> int:
        return self._lib.plh_cache_length(self._book, self._known(request))

    def pages_needed(self, request, new_len: int) -> int:
        """Pages `reserve(request, new_len)` would take, summed over groups."""
        return self._lib.plh_cache_pages_needed(self._book, self._known(request), new_len)

    def reserve(self, request, new_len: int) -> bool:
        """Pages so that tokens [0, new_len) have a place in every group. Takes all
        that is missing or nothing; False when some pool has too few free pages."""
        code = self._lib.plh_cache_reserve(self._book, self._known(request), new_len)
        if code == core.SHRINK:
            raise CacheError(f"request {request!r} cannot shrink from {self.length(request)} to {new_len} tokens")
        if code < 0:
            raise CacheError(f"request {request!r}: reserve({new_len}) failed with code {code}")
        return code == core.OK

    def commit(self, request, new_len: int) -> None:
        """Records that tokens [0, new_len) are cached; gives back the pages of
        windowed groups that no later query can reach."""
        code = self._lib.plh_cache_commit(self._book, self._known(request), new_len)
        if code == core.NOT_RESERVED:
            raise CacheError(f"request {request!r}: commit({new_len}) without pages reserved")
        if code == core.BAD_PAGE:
            raise PageError(f"request {request!r}: a page was given back twice")
        if code < 0:
            raise CacheError(f"request {request!r}: commit({new_len}) failed with code {code}")

    def reserve_many(self, requests: list, n_new: list[int]) -> tuple[np.ndarray, np.ndarray, int]:
        """A step's entries in one call of the host core: for open requests, in order, the
        tokens each holds (int64) and its slot (int32), and pages reserved for n_new[i] more.
        Returns (lengths, slots, done): done == len(requests), or the index of the first
        request for which too few pages were free (what the earlier ones reserved stays)."""
        n = len(requests)
        handles = np.array([self._handles.get(r, -1) for r in requests], dtype=np.int64)
        new = np.asarray(n_new, dtype=np.int32)
        lens = np.empty(n, dtype=np.int64)
        slots = np.empty(n, dtype=np.int32)
        code = ctypes.c_int32(0)
        done = self._lib.plh_cache_reserve_many(self._book, handles.ctypes.data, new.ctypes.data, n, lens.ctypes.data,
                                                slots.ctypes.data, ctypes.byref(code))
        if done < n and code.value != core.NO_ROOM:
            if code.value == core.UNKNOWN_REQUEST:
                raise KeyError(requests[done])
            if code.value == core.SHRINK:
                raise CacheError(f"request {requests[done]!r} cannot shrink")
            raise CacheError(f"request {requests[done]!r}: reserve failed with code {code.value}")
        return lens, slots, done

    def commit_many(self, requests: list, new_lens: list[int]) -> None:
        """commit(request, new_len) for a step's entries in one call of the host core."""
        handles = np.array([self._handles.get(r, -1) for r in requests], dtype=np.int64)
        lens = np.asarray(new_lens, dtype=np.int64)
        code = self._lib.plh_cache_commit_many(self._book, handles.ctypes.data, lens.ctypes.data, len(requests))
        if code == core.NOT_RESERVED:
            raise CacheError("commit without pages reserved")
        if code == core.BAD_PAGE:
            raise PageError("a page was given back twice")
        if code < 0:
            raise CacheError(f"commit failed with code {code}")

    def close(self, request) -> None:
        """Gives back every page and the slot of the request."""
        code = self._lib.plh_cache_close(self._book, self._known(request))
        self.forget(request)
        if code == core.BAD_PAGE:
            raise PageError(f"request {request!r}: a page was given back twice")

    def open_requests(self) -> list:
        out = (ctypes.c_int64 * self.max_requests)()
        n = self._lib.plh_cache_open_requests(self._book, out, self.max_requests)
        return [self._keys[h] for h in out[:n]]

    # ------------------------------------------------------------------ tables
    def table_rows(self, group: int, requests: list, width_multiple: int = 8) -> np.ndarray:
        """int32 [len(requests), W]: each request's page ids of `group`, -1 where it
        holds none; W is the longest row rounded up to `width_multiple`."""
        handles = [self._known(r) for r in requests]
        longest = 1
        for h in handles:
            longest = max(longest, self._lib.plh_cache_table_row(self._book, group, h, self._row, 0))
        width = -(-longest // width_multiple) * width_multiple
        table = np.empty((len(handles), width), dtype=np.int32)
        self.fill_tables(group, handles, table, None)
        return table

    def fill_tables(self, group: int, handles: list[int], table: np.ndarray, slots: np.ndarray | None) -> int:
        """Writes the block-table rows of `handles` into `table` (int32 [n, W], C order;
        -1 where no page) and their slots into `slots`; returns the longest row."""
        n = len(handles)
        ids = (ctypes.c_int64 * max(1, n))(*handles)
        longest = self._lib.plh_cache_fill_tables(
            self._book, group, ids, n, table.ctypes.data_as(ctypes.c_void_p), table.shape[1],
            slots.ctypes.data_as(ctypes.c_void_p) if slots is not None else None)
        if longest < 0:
            raise CacheError(f"fill_tables failed with code {longest}")
        if longest > table.shape[1]:
            raise CacheError(f"a block-table row of {longest} pages does not fit the table's width {table.shape[1]}")
        return longest

    def held_pages(self, request, group: int) -> list[int]:
        n = self._lib.plh_cache_held_pages(self._book, group, self._known(request), self._row, len(self._row))
        return list(self._row[:n])

    # ------------------------------------------------------------------ attention mass
    def take_fresh_pages(self, group: int) -> list[int]:
        """Pages of `group` taken since the last call: their accumulators hold a former
        owner's sums until the next fold clears them."""
        n = self._lib.plh_cache_take_fresh(self._book, group, self._row, len(self._row))
        return list(self._row[:n])

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
            "slots_used": self._lib.plh_cache_slots_used(self._book),
        }

    def free_pages(self) -> int:
        """Free pages of the fullest pool (what limits the next reservation)."""
        return self._lib.plh_cache_free_pages(self._book) if self.groups else self.n_pages
