"""Arrangements of norms, mixer and feed-forward around the residual stream.

A block's forward takes the fp32 residual stream `x` and the previous block's
not-yet-added output `delta`, and returns the same pair: the add is done inside
the next norm kernel (one pass over x instead of two).
"""

from __future__ import annotations

import torch

from . import native_layer
from .registry import BuildContext, build_part, register_part
from .spec import LayerSpec


@register_part("block", "pre_norm")
class PreNormBlock:
    """x += mixer(norm_mixer(x)); x += feed_forward(norm_ff(x))
    (pulsarlm-core/src/engine/model/llama.cpp:88-92). Norm names in the
    LayerSpec: "mixer" and "feed_forward"."""

    def __init__(self, spec: LayerSpec, ctx: BuildContext):
        self.spec = spec
        self.mixer_norm = build_part("norm", spec.norms["mixer"], ctx)
        self.mixer = build_part("mixer", spec.mixer, ctx)
        self.ff_norm = build_part("norm", spec.norms["feed_forward"], ctx)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, ctx)
        self._native: bool | None = None  # whether the parts are the ones the native layer call takes

    @classmethod
    def part_specs(cls, spec: LayerSpec):
        """(kind, PartSpec) of every part, so tensor needs can be listed without building."""
        return [("norm", spec.norms["mixer"]), ("mixer", spec.mixer),
                ("norm", spec.norms["feed_forward"]), ("feed_forward", spec.feed_forward)]

    def parts(self):
        return [self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward]

    def forward(self, x: torch.Tensor, delta: torch.Tensor | None, batch) -> tuple[torch.Tensor, torch.Tensor]:
        # The standard parts in bfloat16: the whole layer from one native call (the same kernels
        # in the same order; see native_layer.py). Anything else: the parts' own calls below.
        if self._native is None:
            self._native = native_layer.eligible(self)
        if self._native:
            done = native_layer.forward(self, x, delta, batch)
            if done is not None:
                return done
        h = self.mixer_norm.forward(x, delta)
        mixed = self.mixer.forward(h, batch)
        h = self.ff_norm.forward(x, mixed)
        return x, self.feed_forward.forward(h, batch)
