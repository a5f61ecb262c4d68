"""The layer launched from one native call (pulsarlm_b200/parts/native_layer.py) against
the same layer launched part by part: the same kernels in the same order, so the same
bits wherever the package's own products run, and the plain implementation's logits
within the usual bar where a library product stands in between."""

import random

import pytest
import torch

import plain_llama
import tiny
from harness import TOLERANCE, record_error
from test_model_gpu import mixed_schedule, replay
from test_schedules_gpu import load, small_config, worst_error

pytestmark = pytest.mark.gpu


def run_schedule(model, reqs, page, native: bool, monkeypatch, graphs: bool = False):
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.engine.runner import ModelRunner
    from pulsarlm_b200.kernels import ops
    from pulsarlm_b200.parts import native_layer

    monkeypatch.setattr(native_layer, "ENABLED", native)
    for block in model.blocks:
        block._native = None
    calls = []
    real = ops.call_native

    def spy(name, *args, **kwargs):
        calls.append(name)
        return real(name, *args, **kwargs)

    monkeypatch.setattr(ops, "call_native", spy)
    lengths = [len(v) for v in reqs.values()]
    n_pages = sum(sorted(-(-n // page) for n in lengths)[-4:])
    runner = ModelRunner(model, CacheManager(model.cache_needs(), page, n_pages, 4, torch.bfloat16, "cuda:0"))
    got = replay(runner, mixed_schedule(reqs, random.Random(11)))
    runner.check_status()
    return got, len(calls)


@pytest.mark.parametrize("head_dim,n_heads,n_kv,page", [(128, 4, 1, 16), (64, 8, 2, 32), (128, 3, 3, 16)])
@pytest.mark.parametrize("route", ["tcgen05", "mixed"])
def test_a_layer_from_one_native_call_equals_the_layer_part_by_part(head_dim, n_heads, n_kv, page, route, monkeypatch):
    from pulsarlm_b200.parts import linear

    monkeypatch.setattr(linear, "GEMM_ROUTE", route)
    cfg = small_config(head_dim, n_heads, n_kv, layers=3)
    weights = tiny.random_weights(cfg, 23, torch.bfloat16)
    model = load(cfg, weights, "bfloat16")
    lengths = [40, 197, 64, 333, 18, 75, 150, 29]
    reqs = {f"r{n}": tiny.random_tokens(cfg, n, seed=500 + n) for n in lengths}
    by_parts, none = run_schedule(model, reqs, page, False, monkeypatch)
    native, calls = run_schedule(model, reqs, page, True, monkeypatch)
    assert none == 0 and calls > 0, "the native layer call was not taken"
    worst = 0.0
    for r, rows in native.items():
        positions = sorted(rows)
        if route == "tcgen05":  # the package's own products on both paths: bit for bit
            for p in positions:
                assert torch.equal(rows[p], by_parts[r][p]), (r, p)
        reference = plain_llama.forward(cfg, weights, reqs[r], dtype=torch.float32)
        err, where = worst_error([rows[p] for p in positions], reference, positions)
        worst = max(worst, err)
        assert err < TOLERANCE["bfloat16"], (r, err, where)
    record_error("bfloat16", f"layers from one native call, head size {head_dim}, route {route}", worst,
                 TOLERANCE["bfloat16"])


def test_other_parts_keep_the_blocks_own_path(monkeypatch):
    """float32, and a layer with a score cap, are not taken by the native call."""
    from pulsarlm_b200.parts import native_layer

    cfg = small_config(64, 4, 2, layers=1)
    weights = tiny.random_weights(cfg, 3, torch.float32)
    model = load(cfg, weights, "float32")
    assert not native_layer.eligible(model.blocks[0])
