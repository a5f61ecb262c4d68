"""Per-page attention-mass accumulators (kept as the reference keeps them; nothing
is evicted here): the attention kernel's sums against the plain definition over
dense scores, through portions, decode tokens, a second request and a reused page."""

import pytest
import torch

import plain_llama
import tiny
from harness import TinyModel

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("key,dtype,tol", [("B", "float32", 1e-4), ("C", "bfloat16", 2e-2)])
def test_attention_mass_matches_dense_scores(key, dtype, tol):
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.engine.loading import load_model
    from pulsarlm_b200.engine.runner import ModelRunner, StepEntry

    tm = TinyModel(key, dtype)
    decay = 0.25
    model = load_model(tm.folder, dtype, "cuda:0")
    cache = CacheManager(model.cache_needs(), tm.page, 12, 2, model.ctx.dtype, "cuda:0", mass_decay=decay)
    runner = ModelRunner(model, cache)
    assert runner.graphs_allowed == (dtype == "bfloat16")  # (the tensor-core decode kernel can measure)

    # an earlier request leaves sums on pages that "a" will then take
    old = tiny.random_tokens(tm.cfg, 70, seed=8)
    runner.step([StepEntry("old", old, [])])
    runner.end("old")

    a = tiny.random_tokens(tm.cfg, 75, seed=1)
    b = tiny.random_tokens(tm.cfg, 20, seed=2)
    portions_a = [(0, 37), (37, 39), (39, 40), (40, 41), (41, 75)]
    runner.step([StepEntry("a", a[0:37], [])])
    runner.step([StepEntry("b", b[0:20], []), StepEntry("a", a[37:39], [])])
    runner.step([StepEntry("a", a[39:40], [])])
    runner.step([StepEntry("a", a[40:41], [])])
    runner.step([StepEntry("a", a[41:75], [])])
    runner.check_status()

    scores: list = []
    plain_llama.forward(tm.cfg, tm.weights, a, scores_out=scores)
    got_mass, got_weight = cache.page_mass("a")
    n_layers = tm.cfg["num_hidden_layers"]
    assert got_mass.shape[0] == n_layers and got_mass.shape[1] == -(-75 // tm.page)
    for layer in range(n_layers):
        want_mass, want_weight = plain_llama.page_attention_mass(scores[layer], portions_a, tm.page, decay)
        assert torch.allclose(got_weight[layer].double().cpu(), want_weight, rtol=1e-5, atol=1e-7), layer
        err = (got_mass[layer].double().cpu() - want_mass).abs().max() / want_mass.abs().max()
        assert err < tol, (layer, float(err))
    # request b was fed in one portion beside a's second one
    scores_b: list = []
    plain_llama.forward(tm.cfg, tm.weights, b, scores_out=scores_b)
    mass_b, weight_b = cache.page_mass("b")
    want_mass, want_weight = plain_llama.page_attention_mass(scores_b[0], [(0, 20)], tm.page, decay)
    assert torch.allclose(weight_b[0].double().cpu(), want_weight, rtol=1e-5, atol=1e-7)
    assert (mass_b[0].double().cpu() - want_mass).abs().max() / want_mass.abs().max() < tol


def test_logits_do_not_change_when_mass_is_measured():
    from pulsarlm_b200 import Engine

    tm = TinyModel("A", "float32")
    prompt = tiny.random_tokens(tm.cfg, 30, seed=4)
    plain = Engine(tm.folder, dtype="float32", n_pages=8, page_size=tm.page)
    measuring = Engine(tm.folder, dtype="float32", n_pages=8, page_size=tm.page, attention_mass_decay=0.1)
    want = plain.generate([prompt], max_tokens=6, ignore_eos=True)
    assert measuring.generate([prompt], max_tokens=6, ignore_eos=True) == want
    assert measuring.runner.graph_steps == 0


@pytest.mark.parametrize("head_dim,n_heads,n_kv,page", [(128, 4, 1, 16), (64, 8, 2, 32)])
def test_attention_mass_from_captured_decode_steps(head_dim, n_heads, n_kv, page):
    """bfloat16 at the tensor-core head sizes: five requests are prefilled (eager steps,
    the CUDA-core kernel measures), then decode through captured steps (padded to eight
    entries), where the tensor-core kernel records each tile's largest score and a fold
    kernel updates the accumulators on the device; one request ends and its pages go to
    a newcomer. Sums per page against the plain definition over dense scores."""
    from harness import record_error
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.engine.runner import ModelRunner, StepEntry
    from pulsarlm_b200.sampling.params import SamplingParams
    from test_schedules_gpu import load, small_config

    cfg = small_config(head_dim, n_heads, n_kv, layers=2)
    weights = tiny.random_weights(cfg, 31, torch.bfloat16)
    model = load(cfg, weights, "bfloat16")
    decay = 0.2
    cache = CacheManager(model.cache_needs(), page, 40, 6, torch.bfloat16, "cuda:0", mass_decay=decay)
    runner = ModelRunner(model, cache)
    assert runner.graphs_allowed
    greedy = SamplingParams(temperature=0.0)
    lengths = {"a": 37, "b": 5, "c": 64, "d": 90, "e": 16}
    n_decode = 40
    tokens = {r: tiny.random_tokens(cfg, n + n_decode, seed=200 + n) for r, n in lengths.items()}
    portions = {r: [(0, n)] for r, n in lengths.items()}
    runner.step([StepEntry(r, tokens[r][:n], []) for r, n in lengths.items()])
    fed = dict(lengths)
    live = list(lengths)
    for step in range(n_decode):
        if step == 12:  # b ends; a newcomer takes its pages and is prefilled in an eager step
            runner.end("b")
            live.remove("b")
            tokens["f"] = tiny.random_tokens(cfg, 20 + n_decode, seed=77)
            runner.step([StepEntry("f", tokens["f"][:20], [])])
            portions["f"], fed["f"] = [(0, 20)], 20
            live.append("f")
        entries = [StepEntry(r, [tokens[r][fed[r]]], [0]) for r in live]
        runner.decode_step(entries, [greedy] * len(live), [0] * len(live), [0] * len(live))
        for r in live:
            portions[r].append((fed[r], fed[r] + 1))
            fed[r] += 1
    runner.check_status()
    assert runner.graph_steps == n_decode and all(n == 8 for n, _ in runner._graphs)
    worst = 0.0
    for r in live:
        scores: list = []
        plain_llama.forward(cfg, weights, tokens[r][: fed[r]], scores_out=scores)
        got_mass, got_weight = cache.page_mass(r)
        for layer in range(cfg["num_hidden_layers"]):
            want_mass, want_weight = plain_llama.page_attention_mass(scores[layer], portions[r], page, decay)
            assert torch.allclose(got_weight[layer].double().cpu(), want_weight, rtol=1e-5, atol=1e-7), (r, layer)
            err = float((got_mass[layer].double().cpu() - want_mass).abs().max() / want_mass.abs().max())
            worst = max(worst, err)
            assert err < 2e-2, (r, layer, err)
    record_error("bfloat16", f"attention mass from captured decode steps, head size {head_dim}", worst, 2e-2)


@pytest.mark.parametrize("head_dim,n_heads,n_kv,page", [(128, 4, 1, 16), (64, 8, 2, 32), (128, 3, 3, 64),
                                                         (64, 4, 2, 16)])
def test_attention_mass_from_prompt_portions_on_the_tensor_cores(head_dim, n_heads, n_kv, page, monkeypatch):
    """bfloat16 at the tensor-core head sizes, eager steps: prompt portions go through the
    tcgen05 kernel, whose softmax warps add up weight * (largest score in the page) over
    their rows, and a fold kernel adds the warps' sums in a fixed order; single tokens beside
    them go through the CUDA-core kernel. Portions that end inside a page and inside a
    64-key tile, two requests in one step, one request's pages taken over by another, an
    odd group (tiles of 256 rows in two halves). Against the plain definition over dense
    scores; the same steps twice give the same bits."""
    from harness import record_error
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.engine.runner import ModelRunner, StepEntry
    from pulsarlm_b200.kernels import ops
    from test_schedules_gpu import load, small_config

    cfg = small_config(head_dim, n_heads, n_kv, layers=2)
    weights = tiny.random_weights(cfg, 17, torch.bfloat16)
    model = load(cfg, weights, "bfloat16")
    decay = 0.05
    measured = []
    real = ops.attention_prefill_tcgen05

    def spy(*args, **kwargs):
        measured.append(kwargs.get("mass") is not None)
        return real(*args, **kwargs)

    monkeypatch.setattr(ops, "attention_prefill_tcgen05", spy)
    a = tiny.random_tokens(cfg, 470, seed=1)
    b = tiny.random_tokens(cfg, 150, seed=2)
    old = tiny.random_tokens(cfg, 200, seed=3)
    portions_a = [(0, 300), (300, 302), (302, 303), (303, 470)]

    def run():
        cache = CacheManager(model.cache_needs(), page, -(-470 // page) + -(-200 // page) + 2, 3, torch.bfloat16,
                             "cuda:0", mass_decay=decay)
        runner = ModelRunner(model, cache)
        runner.step([StepEntry("old", old, [])])
        runner.step([StepEntry("a", a[0:300], [])])
        runner.end("old")  # its pages, with its sums on them, go to b and to the rest of a
        runner.step([StepEntry("b", b[0:150], []), StepEntry("a", a[300:302], [])])
        runner.step([StepEntry("a", a[302:303], []), StepEntry("b", b[150:], [])] if len(b) > 150 else
                    [StepEntry("a", a[302:303], [])])
        runner.step([StepEntry("a", a[303:470], [])])
        runner.check_status()
        return cache.page_mass("a"), cache.page_mass("b")

    (mass_a, weight_a), (mass_b, weight_b) = run()
    assert any(measured), "no prompt portion was measured by the tcgen05 kernel"
    worst = 0.0
    for tokens, portions, got_mass, got_weight in ((a, portions_a, mass_a, weight_a), (b, [(0, 150)], mass_b, weight_b)):
        scores: list = []
        plain_llama.forward(cfg, weights, tokens, scores_out=scores)
        for layer in range(cfg["num_hidden_layers"]):
            want_mass, want_weight = plain_llama.page_attention_mass(scores[layer], portions, page, decay)
            assert torch.allclose(got_weight[layer].double().cpu(), want_weight, rtol=1e-4, atol=1e-7), layer
            err = float((got_mass[layer].double().cpu() - want_mass).abs().max() / want_mass.abs().max())
            worst = max(worst, err)
            assert err < 2e-2, (layer, err)
    record_error("bfloat16", f"attention mass from tcgen05 prompt portions, head size {head_dim}, page {page}", worst,
                 2e-2)
    (again_a, again_wa), _ = run()
    assert torch.equal(again_a, mass_a) and torch.equal(again_wa, weight_a)
