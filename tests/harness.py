"""Helpers of the GPU tests: build a runner over a tiny model, replay schedules,
compare with the plain implementation."""

from __future__ import annotations

import tempfile

import torch

import plain_llama
import tiny

# The reference's own bars for its Llama test (pulsarlm-core/tests/model/test_llama.cpp:
# 278-289): 1e-4 in fp32 and 1e-2 in bf16, max|difference| / max|expected|. (bf16
# started at 2e-2 here and was tightened once every comparison printed its worst error:
# the largest seen is 7.4e-3, fp32 stays below 1e-6; the run's summary lists them.)
TOLERANCE = {"float32": 1e-4, "bfloat16": 1e-2}

# (dtype, what) -> (worst relative error seen in this run, the bar it was held to)
WORST: dict = {}


def record_error(dtype: str, what: str, err: float, bar: float) -> None:
    """Remembers the worst error of a kind of comparison; printed at the end of the run."""
    key = (dtype, what)
    if key not in WORST or err > WORST[key][0]:
        WORST[key] = (err, bar)


CONFIGS = {
    "A": (tiny.TINY_A, tiny.PAGE_A),
    "B": (tiny.TINY_B, tiny.PAGE_B),
    "C": (tiny.TINY_C, tiny.PAGE_C),
}


def torch_dtype(name: str) -> torch.dtype:
    return torch.float32 if name == "float32" else torch.bfloat16


class TinyModel:
    """A tiny config with random weights (rounded to the engine dtype, so the plain
    implementation and the engine start from identical numbers), a model folder,
    and the plain implementation's logits on demand."""

    def __init__(self, key: str, dtype: str, seed: int = 1):
        self.cfg, self.page = CONFIGS[key]
        self.dtype = dtype
        self.weights = tiny.random_weights(self.cfg, seed, torch_dtype(dtype))
        self._dir = tempfile.TemporaryDirectory()
        self.folder = tiny.write_model_dir(self._dir.name, self.cfg, self.weights)
        self._plain: dict[tuple, torch.Tensor] = {}

    def plain_logits(self, tokens) -> torch.Tensor:
        key = tuple(tokens)
        if key not in self._plain:
            self._plain[key] = plain_llama.forward(self.cfg, self.weights, list(tokens))
        return self._plain[key]

    def runner(self, n_pages: int, slots: int = 4, page: int | None = None):
        from pulsarlm_b200.cache.manager import CacheManager
        from pulsarlm_b200.engine.loading import load_model
        from pulsarlm_b200.engine.runner import ModelRunner

        model = load_model(self.folder, self.dtype, "cuda:0")
        cache = CacheManager(model.cache_needs(), page or self.page, n_pages, slots, model.ctx.dtype, "cuda:0")
        return ModelRunner(model, cache)


def replay(runner, steps) -> dict:
    """steps: list of (entries, ends); entries = [(request, tokens, want)]. Returns
    {request: {position: logits row}} with positions counted within the request."""
    from pulsarlm_b200.engine.runner import StepEntry

    fed: dict = {}
    out: dict = {}
    for entries, ends in steps:
        step_entries = [StepEntry(r, list(t), list(w)) for r, t, w in entries]
        logits = runner.step(step_entries)
        row = 0
        for r, t, w in entries:
            start = fed.get(r, 0)
            for place in w:
                out.setdefault(r, {})[start + place] = logits[row].float().cpu()
                row += 1
            fed[r] = start + len(t)
        for r in ends:
            runner.end(r)
            fed.pop(r, None)
    runner.check_status()
    return out


def assert_matches_plain(tm: TinyModel, request_tokens: dict, got: dict, what: str) -> float:
    """Every returned row against the plain implementation's row at that position."""
    worst = 0.0
    for r, rows in got.items():
        ref = tm.plain_logits(request_tokens[r])
        positions = sorted(rows)
        g = torch.stack([rows[p] for p in positions])
        e = ref[positions]
        err = plain_llama.max_relative_error(g, e)
        worst = max(worst, err)
        if not err < TOLERANCE[tm.dtype]:
            per_row = (g.double() - e).abs().amax(dim=1) / e.abs().max()
            first = positions[int(torch.nonzero(per_row >= TOLERANCE[tm.dtype])[0, 0])]
            raise AssertionError(f"{what}: request {r!r} differs from the plain implementation: max rel error "
                                 f"{err:.3e} (bar {TOLERANCE[tm.dtype]:.0e}); first wrong position {first} "
                                 f"of {len(request_tokens[r])}")
    record_error(tm.dtype, what, worst, TOLERANCE[tm.dtype])
    return worst
