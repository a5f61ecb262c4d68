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
    assert not runner.graphs_allowed

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
