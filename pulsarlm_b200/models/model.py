"""The generic model: parts built from a ModelSpec and run in the spec's order.

Nothing here is specific to an architecture. The model owns no cache; the cache
manager asks `cache_needs()` what each layer wants and hands bindings back
through `bind_caches()`.
"""

from __future__ import annotations

import dataclasses

import torch

from ..parts import attention, basic, block  # noqa: F401  (registers the built-in parts)
from ..parts.registry import BuildContext, build_part, part_class
from ..parts.spec import ModelSpec, TensorNeed


@dataclasses.dataclass
class StepBatch:
    """One step's tokens, on the device.

    tokens, pos, entry: int32 [T]; token t is `tokens[t]` at position `pos[t]` of
    the request in batch entry `entry[t]`. tables[g]: int32 [entries, width], the
    block-table rows of cache group g for this step's entries. slots: int32
    [entries], each entry's state slot. want_rows: int32 [R], indices into the T
    tokens whose logits are wanted (None: none). status: int32 [1] that kernels
    OR error bits into. Entries of a single token come first: the leading `n_decode`
    tokens are each the one token of their entry. The host_* fields repeat sizes
    for kernels' launchers.
    """

    tokens: torch.Tensor
    pos: torch.Tensor
    entry: torch.Tensor
    tables: dict[int, torch.Tensor]
    slots: torch.Tensor
    want_rows: torch.Tensor | None
    status: torch.Tensor
    n_tokens: int
    n_entries: int
    n_decode: int = 0
    host_query_lens: list[int] = dataclasses.field(default_factory=list)
    host_context_lens: list[int] = dataclasses.field(default_factory=list)
    extras: dict = dataclasses.field(default_factory=dict)
    # What the parts planned for this step on the host (see HostStep): plans[key][name]
    # is a device tensor for every array a part's plan_step returned under `name`, and
    # the value itself for everything else. `key` is the part's plan_key().
    plans: dict = dataclasses.field(default_factory=dict)


@dataclasses.dataclass
class HostStep:
    """What the host knows of a step before it runs: the sizes of its entries, in batch
    order (entries of one token first). Parts that need index arrays of their own for
    a step (tile lists, chunk boundaries, expert offsets) build them from this in
    `plan_step`; the step function stages what they return with its own arrays and
    hands it back in `StepBatch.plans`.

    query_lens[e]: tokens of entry e in this step. context_lens[e]: tokens its
    request holds after the step. first_rows[e]: row of its first token among the
    step's tokens. A step that is captured once and replayed (`fixed_shape`) is
    planned anew before every replay: the arrays a part returns must then have shapes
    that depend only on n_entries and context_bound (the most tokens any entry of a
    replay may hold), and what it returns besides arrays is kept from the first call,
    so it must depend on nothing else either. A part that wants different kernels for
    different replays of one shape (say, for requests of equal and of unequal lengths)
    answers `plan_variant(step)` with a hashable value: replays whose values differ get
    captures of their own, and `variants[part.plan_key()]` holds the value the capture
    at hand was made for."""

    n_entries: int
    n_tokens: int
    n_decode: int
    query_lens: list[int]
    context_lens: list[int]
    first_rows: list[int]
    page_size: int
    fixed_shape: bool = False
    context_bound: int | None = None
    variants: dict = dataclasses.field(default_factory=dict)


def _all_part_specs(spec: ModelSpec):
    yield "embedding", spec.embedding
    for layer in spec.layers:
        yield from part_class("block", layer.block).part_specs(layer)
    yield "norm", spec.final_norm
    yield "head", spec.head


def tensor_needs_of(spec: ModelSpec) -> dict[str, TensorNeed]:
    """Every checkpoint tensor the model's parts need, by name. A name two parts
    ask for must be asked for with the same shape."""
    needs: dict[str, TensorNeed] = {}
    for kind, part_spec in _all_part_specs(spec):
        for name, need in part_class(kind, part_spec.kind).tensor_needs(part_spec).items():
            if name in needs and needs[name].shape != need.shape:
                raise ValueError(f"tensor {name!r} is needed with shapes {needs[name].shape} and {need.shape}")
            needs.setdefault(name, need)
    return needs


class Model:
    """Embedding, blocks in `spec.order`, final norm, head."""

    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"engine dtype must be float32 or bfloat16, got {dtype}")
        self.spec = spec
        self.ctx = BuildContext(dtype=dtype, device=torch.device(device))
        for index in spec.order:
            if not 0 <= index < len(spec.layers):
                raise ValueError(f"layer order names layer {index}, but there are {len(spec.layers)} layers")
        self.embedding = build_part("embedding", spec.embedding, self.ctx)
        self.blocks = [part_class("block", layer.block)(layer, self.ctx) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, self.ctx)
        self.head = build_part("head", spec.head, self.ctx)
        self.loaded = False

    # ------------------------------------------------------------------ weights
    def tensor_needs(self) -> dict[str, TensorNeed]:
        return tensor_needs_of(self.spec)

    def parts(self):
        yield self.embedding
        for b in self.blocks:
            yield from b.parts()
        yield self.final_norm
        yield self.head

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        """`tensors`: checked, converted, on the device (see weights.loader)."""
        for part in self.parts():
            part.load(tensors)
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding.weight)
        self.loaded = True

    # ------------------------------------------------------------------ cache
    def cache_needs(self) -> list:
        """Per layer: the mixer's KVCacheNeed, StateNeed or None."""
        return [b.mixer.cache_need() for b in self.blocks]

    def cache_sources(self) -> list[int | None]:
        """Per layer: the layer whose cache it reads instead of its own, or None."""
        sources = [getattr(b.mixer, "cache_from", None) for b in self.blocks]
        needs = self.cache_needs()
        for layer, src in enumerate(sources):
            if src is None:
                continue
            if not 0 <= src < len(self.blocks) or needs[src] is None or sources[src] is not None:
                raise ValueError(f"layer {layer} reads the cache of layer {src}, which keeps none of its own")
            # The reader must see the cache as its owner keeps it: the same heads and head
            # size, and no further back than the owner's window (pages behind that window
            # are given back while the request runs).
            reads = getattr(self.blocks[layer].mixer, "cache_read_need", None)
            want, have = (reads() if reads is not None else None), needs[src]
            if want is not None and hasattr(have, "n_kv_heads"):
                if (want.n_kv_heads, want.head_dim) != (have.n_kv_heads, have.head_dim):
                    raise ValueError(
                        f"layer {layer} reads the cache of layer {src} as {want.n_kv_heads} kv heads of size "
                        f"{want.head_dim}, but it holds {have.n_kv_heads} of size {have.head_dim}")
                if have.window is not None and (want.window is None or want.window > have.window):
                    raise ValueError(
                        f"layer {layer} reads {'every key' if want.window is None else f'a window of {want.window}'} "
                        f"of layer {src}'s cache, which keeps a window of {have.window} only")
        return sources

    def planners(self) -> list:
        """The parts that plan steps on the host, one per distinct plan_key()."""
        seen: dict = {}
        for part in self.parts():
            key_of = getattr(part, "plan_key", None)
            key = key_of() if key_of is not None else None
            if key is not None and key not in seen:
                seen[key] = part
        return list(seen.items())

    def bind_caches(self, bindings: list) -> None:
        sources = self.cache_sources()
        for layer, b in enumerate(self.blocks):
            src = sources[layer] if sources[layer] is not None else layer
            if bindings[src] is not None:
                b.mixer.bind_cache(bindings[src])

    # ------------------------------------------------------------------ forward
    def forward(self, batch: StepBatch) -> torch.Tensor | None:
        """Runs the batch's tokens through every layer in order; returns fp32 logits
        [R, vocab] at `batch.want_rows`, or None when none are wanted."""
        if not self.loaded:
            raise RuntimeError("the model has no weights loaded")
        x = self.embedding.forward(batch.tokens, batch)
        delta = None
        for index in self.spec.order:
            x, delta = self.blocks[index].forward(x, delta, batch)
        if batch.want_rows is None or batch.want_rows.numel() == 0:
            return None
        h = self.final_norm.forward(x, delta, rows=batch.want_rows)
        return self.head.forward(h)
