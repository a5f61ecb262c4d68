"""Per-request sampling options, with the reference's names, meanings and defaults
(pulsarlm-core/inc/pulsarlm/engine/sampling_params.hpp:11-16)."""

from __future__ import annotations

import dataclasses
import secrets


@dataclasses.dataclass(frozen=True)
class SamplingParams:
    """temperature <= 0 takes the argmax (ties to the lower id). top_p outside
    (0, 1) and top_k = 0 are off. seed None draws a fresh seed per request; with
    a seed, the tokens are a pure function of (seed, how many tokens the request
    has drawn, the logits)."""

    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    seed: int | None = None

    def __post_init__(self):
        if self.temperature != self.temperature or self.temperature < 0.0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if self.top_p != self.top_p:
            raise ValueError("top_p must be a number")

    @property
    def draws(self) -> bool:
        return self.temperature > 0.0

    def resolved_seed(self) -> int:
        """The request's 64-bit seed (pulsarlm-core/src/engine/sampling.cpp:30-36)."""
        if self.seed is not None:
            return int(self.seed) & 0xFFFFFFFFFFFFFFFF
        return secrets.randbits(64)
