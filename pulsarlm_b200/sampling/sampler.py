"""Host side of sampling: per-row options to device arrays, one kernel launch.

The reference builds per-row tensors the same way and races Gumbel noise over
the logits (pulsarlm-core/src/engine/sampling.cpp:40-76)."""

from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams


def _signed64(value: int) -> int:
    value &= 0xFFFFFFFFFFFFFFFF
    return value - (1 << 64) if value >= (1 << 63) else value


class Sampler:
    def __init__(self, device: torch.device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, params: list[SamplingParams], seeds: list[int],
               draw_counts: list[int]) -> torch.Tensor:
        """int32 [rows] on the device: one token per row of fp32 logits [rows, vocab].
        seeds[r] and draw_counts[r] key row r's noise."""
        rows = logits.shape[0]
        if not (len(params) == len(seeds) == len(draw_counts) == rows):
            raise ValueError("one SamplingParams, seed and draw count per row of logits")
        floats = np.empty((2, rows), dtype=np.float32)
        ints = np.empty((rows,), dtype=np.int32)
        longs = np.empty((2, rows), dtype=np.int64)
        any_filter = False
        for r, p in enumerate(params):
            floats[0, r] = p.temperature if p.draws else 0.0
            keeps_p = 0.0 < p.top_p < 1.0
            floats[1, r] = p.top_p if keeps_p else 2.0
            ints[r] = p.top_k
            any_filter |= p.draws and (keeps_p or p.top_k > 0)
            longs[0, r] = _signed64(seeds[r])
            longs[1, r] = _signed64(draw_counts[r])
        f = torch.from_numpy(floats).to(self.device, non_blocking=True)
        l = torch.from_numpy(longs).to(self.device, non_blocking=True)
        i = torch.from_numpy(ints).to(self.device, non_blocking=True) if any_filter else None
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        ops.sample(logits, f[0], i, f[1] if any_filter else None, l[0], l[1], out)
        return out
