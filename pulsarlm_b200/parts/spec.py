"""A model as data: which parts, with which sizes, reading which tensors, in which order.

An architecture's `describe(config)` returns a ModelSpec. The generic model
(pulsarlm_b200/models/model.py) builds parts from it through the part
registries; no part learns which architecture it sits in.
"""

from __future__ import annotations

import dataclasses
from typing import Any


@dataclasses.dataclass
class PartSpec:
    """One part: `kind` selects the class in its registry, `params` are its sizes
    and constants, `tensors` maps the part's own role names (e.g. "q", "gate")
    to tensor names in the checkpoint. A role mapped to None is absent (e.g. a
    tied head has no tensor of its own)."""

    kind: str
    params: dict[str, Any] = dataclasses.field(default_factory=dict)
    tensors: dict[str, str | None] = dataclasses.field(default_factory=dict)


@dataclasses.dataclass
class LayerSpec:
    """One layer: an arrangement (`block`, e.g. "pre_norm") of a mixer, a
    feed-forward and the norms the arrangement names."""

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: dict[str, PartSpec]


@dataclasses.dataclass
class ModelSpec:
    """The whole model. `order` lists layer indices in the order they run; an
    index may appear twice (the layer then runs twice with the same weights and
    cache). A mixer whose params hold `cache_from = k` reads (and does not
    write) the cache of layer k."""

    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: list[LayerSpec]
    order: list[int]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: tuple[int, ...] = ()
    max_position_embeddings: int | None = None


@dataclasses.dataclass(frozen=True)
class TensorNeed:
    """What a part expects of one checkpoint tensor. `role` is "matrix" for
    operands of matrix products and embedding tables (converted to the engine's
    dtype) or "vector" for scales and the like (a tensor stored in 32-bit stays
    32-bit) or "ignored" for a tensor that may be stored but is not read.
    `optional` tensors may be missing."""

    shape: tuple[int, ...]
    role: str = "matrix"
    optional: bool = False


@dataclasses.dataclass(frozen=True)
class KVCacheNeed:
    """A mixer that keeps keys and values: per token `n_kv_heads * head_dim` keys
    and as many values. `window` = None keeps every token; a number keeps only the
    last `window` tokens readable, and pages wholly before them are given back.
    `n_heads` is the number of query heads that read the cache; the cache manager
    sizes the optional per-page attention-mass accumulators by it."""

    n_kv_heads: int
    head_dim: int
    window: int | None = None
    n_heads: int = 0


@dataclasses.dataclass(frozen=True)
class StateNeed:
    """A mixer that keeps a state of fixed size per request: `shape` elements of
    `dtype` ("float32" or "bfloat16"), zeroed when a request gets its slot."""

    shape: tuple[int, ...]
    dtype: str = "float32"
