"""Registries of part classes, one per kind of part, and the interfaces parts keep.

A part class is registered under a name and built from a PartSpec:

    part = build_part("mixer", spec, ctx)        # ctx: BuildContext (dtype, device)

Interfaces (duck-typed; the base classes below document them):

* every part:  `tensor_needs(spec) -> {checkpoint name: TensorNeed}` (classmethod),
               `load(tensors)` with the checked tensors, by checkpoint name.
               Optionally `plan_key()` and `plan_step(host_step)`: a part that needs
               index arrays of its own for a step returns them (numpy int32 or
               float32 arrays, by name) from `plan_step`; the step function copies
               them to the device with its own arrays and the part finds them in
               `batch.plans[plan_key()]`. Parts with equal keys share one plan.
* embedding:   `forward(tokens, batch) -> x` fp32 [T, H].
* norm:        `forward(x, delta=None, rows=None) -> h`: x is the fp32 residual
               stream [T, H]; `delta` (engine dtype) is first added into x in
               place; `rows` (int32) selects rows instead of running all.
* position:    owned by the mixer that uses it; `table()` gives what its kernel
               needs.
* mixer:       `cache_need() -> KVCacheNeed | StateNeed | None`,
               `bind_cache(binding)`, `forward(h, batch) -> [T, H]` engine dtype.
* feed_forward:`forward(h, batch) -> [T, H]` engine dtype.
* block:       `forward(x, delta, batch) -> (x, delta)`: the arrangement of
               norms, mixer and feed-forward around the residual stream.
"""

from __future__ import annotations

import dataclasses
from typing import Any

import torch

from .spec import PartSpec, TensorNeed

_KINDS = ("norm", "position", "mixer", "feed_forward", "block", "embedding", "head")
_REGISTRIES: dict[str, dict[str, type]] = {k: {} for k in _KINDS}


@dataclasses.dataclass
class BuildContext:
    """What every part is told when built: the engine's dtype and device."""

    dtype: torch.dtype
    device: torch.device


def register_part(kind: str, name: str, cls: type | None = None, replace: bool = False):
    """Registers `cls` as the part `name` of `kind`; usable as a decorator."""
    if kind not in _REGISTRIES:
        raise ValueError(f"unknown kind of part {kind!r}; kinds: {', '.join(_KINDS)}")

    def add(c: type) -> type:
        if name in _REGISTRIES[kind] and not replace:
            raise ValueError(f"{kind} {name!r} is already registered")
        _REGISTRIES[kind][name] = c
        return c

    return add if cls is None else add(cls)


_builtins_loaded = False


def _load_builtins() -> None:
    """The package's own parts register themselves when their modules are imported."""
    global _builtins_loaded
    if not _builtins_loaded:
        _builtins_loaded = True
        from . import attention, basic, block  # noqa: F401


def part_class(kind: str, name: str) -> type:
    _load_builtins()
    try:
        return _REGISTRIES[kind][name]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES.get(kind, {}))) or "none"
        raise ValueError(f"no {kind} named {name!r} is registered (known: {known})") from None


def build_part(kind: str, spec: PartSpec, ctx: BuildContext, **extra: Any):
    return part_class(kind, spec.kind)(spec, ctx, **extra)


def registered_parts(kind: str) -> list[str]:
    _load_builtins()
    return sorted(_REGISTRIES[kind])


class Part:
    """Base of all parts: keeps the spec and the build context."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        self.spec = spec
        self.ctx = ctx

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        return {}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        pass

    def plan_key(self):
        """A hashable naming this part's per-step plan, or None when it plans nothing.
        Parts that return equal keys (the same mixer in every layer) are planned once."""
        return None

    def plan_step(self, step) -> dict:
        """Host-side planning of one step (see models.model.HostStep): arrays by name,
        and anything else the part wants to find in `batch.plans[plan_key()]`."""
        return {}

    def param(self, name: str):
        try:
            return self.spec.params[name]
        except KeyError:
            raise ValueError(f"{type(self).__name__}: spec lacks the parameter {name!r}") from None
