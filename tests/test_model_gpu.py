"""The engine against the plain implementation, in float32 and bfloat16, under every
way of cutting the work: whole, tail one by one, portions of changing size, mixed
batches with page reuse, long decoding, the first tokens of a sequence."""

import random

import pytest
import torch

import tiny
from harness import CONFIGS, TinyModel, assert_matches_plain, replay

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
KEYS = ["A", "B", "C"]
LENGTHS = [5, 17, 33, 70, 100, 200]

_models: dict = {}


def tiny_model(key, dtype) -> TinyModel:
    if (key, dtype) not in _models:
        _models[(key, dtype)] = TinyModel(key, dtype)
    return _models[(key, dtype)]


def prompts(tm, lengths=LENGTHS):
    return {f"r{n}": tiny.random_tokens(tm.cfg, n, seed=100 + n) for n in lengths}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", KEYS)
def test_each_request_alone_and_whole(key, dtype):
    tm = tiny_model(key, dtype)
    reqs = prompts(tm)
    runner = tm.runner(n_pages=16)
    steps = [([(r, t, range(len(t)))], [r]) for r, t in reqs.items()]
    assert_matches_plain(tm, reqs, replay(runner, steps), "whole")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", KEYS)
def test_last_32_tokens_one_by_one(key, dtype):
    tm = tiny_model(key, dtype)
    reqs = prompts(tm, [33, 70, 200])
    runner = tm.runner(n_pages=16)
    steps = []
    for r, t in reqs.items():
        head = len(t) - 32
        steps.append(([(r, t[:head], range(head))], []))
        for i in range(head, len(t)):
            steps.append(([(r, t[i:i + 1], [0])], [r] if i == len(t) - 1 else []))
    assert_matches_plain(tm, reqs, replay(runner, steps), "tail one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", KEYS)
def test_portions_of_changing_size(key, dtype):
    tm = tiny_model(key, dtype)
    reqs = prompts(tm, [70, 100, 200])
    runner = tm.runner(n_pages=16)
    for sizes in ([13], [2, 5, 3, 17, 2, 31, 7], [2]):
        steps = []
        for r, t in reqs.items():
            at, i = 0, 0
            while at < len(t):
                n = min(sizes[i % len(sizes)], len(t) - at)
                if len(t) - at - n == 1:
                    n += 1  # no portion of one token here: that is the decode path's test
                i += 1
                steps.append(([(r, t[at:at + n], range(n))], [r] if at + n == len(t) else []))
                at += n
        assert_matches_plain(tm, reqs, replay(runner, steps), f"portions {sizes}")


def mixed_schedule(reqs: dict, rng: random.Random, live_limit=4):
    """Up to four live requests; each step every live request feeds either one token
    (a decode) or a portion of 2..24, some sit a step out; a finished request ends
    and the next one starts, so its pages are used again."""
    waiting = list(reqs)
    live: dict = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < live_limit:
            live[waiting.pop(0)] = 0
        entries, ends = [], []
        for r in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue
            at = live[r]
            left = len(reqs[r]) - at
            n = 1 if rng.random() < 0.5 else rng.randrange(2, 25)
            n = min(n, left)
            want = range(n) if rng.random() < 0.7 else ([n - 1] if rng.random() < 0.5 else [])
            entries.append((r, reqs[r][at:at + n], want))
            live[r] = at + n
            if live[r] == len(reqs[r]):
                ends.append(r)
                del live[r]
        if entries:
            rng.shuffle(entries)
            steps.append((entries, ends))
    return steps


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", KEYS)
def test_mixed_batches_with_page_reuse(key, dtype):
    tm = tiny_model(key, dtype)
    lengths = [40, 97, 64, 33, 120, 18, 75, 50, 101, 29]
    reqs = prompts(tm, lengths)
    page = tm.page
    # Room for the four longest at once and not a page more: every later request
    # lands on pages another request has used.
    n_pages = sum(sorted(-(-n // page) for n in lengths)[-4:])
    runner = tm.runner(n_pages=n_pages, slots=4)
    steps = mixed_schedule(reqs, random.Random(11))
    got = replay(runner, steps)
    assert runner.cache.groups[0].pool.high_water > n_pages // 2
    assert_matches_plain(tm, reqs, got, "mixed")
    assert runner.cache.free_pages() == n_pages


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", ["B", "C"])
def test_long_decoding(key, dtype):
    tm = tiny_model(key, dtype)
    n = 420
    reqs = {"long": tiny.random_tokens(tm.cfg, n, seed=9)}
    t = reqs["long"]
    runner = tm.runner(n_pages=-(-n // tm.page))
    steps = [([("long", t[:4], range(4))], [])]
    steps += [([("long", t[i:i + 1], [0])], []) for i in range(4, n)]
    assert_matches_plain(tm, reqs, replay(runner, steps), "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", KEYS)
def test_first_tokens_of_a_sequence(key, dtype):
    tm = tiny_model(key, dtype)
    reqs = prompts(tm, [1, 2, 3])
    runner = tm.runner(n_pages=8)
    steps = [([(r, t[:1], [0])], []) for r, t in reqs.items()]
    steps += [([(r, t[1:], range(len(t) - 1)) for r, t in reqs.items() if len(t) > 1], list(reqs))]
    assert_matches_plain(tm, reqs, replay(runner, steps), "first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_cutting_does_not_change_float32_bits_and_barely_bfloat16(dtype):
    """The same request cut three ways: in float32 every kernel adds in an order
    that does not depend on the batch, so the logits are identical bit for bit."""
    tm = tiny_model("B", dtype)
    t = tiny.random_tokens(tm.cfg, 90, seed=5)
    runner = tm.runner(n_pages=8)
    whole = replay(runner, [([("r", t, range(90))], ["r"])])["r"]
    cut = replay(runner, [([("r", t[:37], range(37))], []), ([("r", t[37:39], range(2))], []),
                          ([("r", t[39:], range(51))], ["r"])])["r"]
    other = tiny.random_tokens(tm.cfg, 30, seed=6)
    beside = replay(runner, [([("o", other[:20], []), ("r", t[:50], range(50))], []),
                             ([("r", t[50:51], [0]), ("o", other[20:], [])], ["o"]),
                             ([("r", t[51:], range(39))], ["r"])])["r"]
    for p in range(90):
        if dtype == "float32":
            assert torch.equal(whole[p], cut[p]) and torch.equal(whole[p], beside[p]), p
        else:
            scale = whole[p].abs().max()
            assert (whole[p] - cut[p]).abs().max() <= 2e-2 * scale, p
            assert (whole[p] - beside[p]).abs().max() <= 2e-2 * scale, p


@pytest.mark.parametrize("route", ["tcgen05", "library"])
@pytest.mark.parametrize("key", KEYS)
def test_every_bfloat16_product_route_gives_the_same_model(key, route, monkeypatch):
    """The default route picks a kernel by the size of the product; the tiny models
    would leave the pair kernel and its SwiGLU epilogue idle. With the route forced,
    every projection of the model runs on the own tcgen05 kernels (skinny up to 64
    tokens, pairs of SMs above, the gate/up projection with the activation in its
    epilogue), or on the library, and the logits still match the plain implementation:
    prompts in one portion, in portions, and single tokens."""
    from pulsarlm_b200.parts import linear

    monkeypatch.setattr(linear, "GEMM_ROUTE", route)
    tm = tiny_model(key, "bfloat16")
    reqs = prompts(tm, [70, 100, 200, 300])
    runner = tm.runner(n_pages=32)
    steps = []
    for r, t in reqs.items():
        if len(t) == 300:  # 130 tokens, then 65, then the rest one by one over the last few
            steps.append(([(r, t[:130], range(130))], []))
            steps.append(([(r, t[130:295], range(165))], []))
            for i in range(295, 300):
                steps.append(([(r, t[i:i + 1], [0])], [r] if i == 299 else []))
        else:
            steps.append(([(r, t, range(len(t)))], [r]))
    assert_matches_plain(tm, reqs, replay(runner, steps), f"route {route}")
