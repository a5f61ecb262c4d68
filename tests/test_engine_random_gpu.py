"""The engine under arrivals, page pressure and cancellations drawn at random (float32,
greedy): whatever the scheduler decides (portions, preemption and recomputation,
pipelined or plain decode steps, graphs or eager), every request that is not cancelled
ends with exactly the tokens the plain implementation generates for it alone."""

import random
import tempfile

import pytest
import torch

import plain_llama
import tiny

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", [1, 3, 5, 9, 14, 16, 40, 77])  # (1, 3, 9, 14 and 16 preempt)
def test_random_arrivals_under_page_pressure(seed):
    from pulsarlm_b200 import Engine, SamplingParams
    from pulsarlm_b200.engine.loading import load_model

    rng = random.Random(seed)
    cfg, page = rng.choice([(tiny.TINY_A, tiny.PAGE_A), (tiny.TINY_B, tiny.PAGE_B)])
    weights = tiny.random_weights(cfg, seed, torch.float32)
    with tempfile.TemporaryDirectory() as folder:
        model = load_model(tiny.write_model_dir(folder, cfg, weights), "float32", "cuda:0")
    n_requests = rng.choice([3, 5, 8])
    prompts = [tiny.random_tokens(cfg, rng.choice([1, 4, 20, 33, 70, 120]), seed * 100 + i) for i in range(n_requests)]
    new_tokens = [rng.choice([1, 3, 9, 20]) for _ in range(n_requests)]
    largest = max(len(p) + n for p, n in zip(prompts, new_tokens))
    n_pages = -(-largest // page) + rng.choice([0, 1, 3, 10, 40])  # sometimes only one request fits at a time
    engine = Engine(model, n_pages=n_pages, page_size=page, prefill_tokens_per_step=rng.choice([2, 7, 32, 256]),
                    max_requests=rng.choice([2, 4, 8]), stop_ids=[], cuda_graphs=rng.random() < 0.7,
                    lookahead=rng.random() < 0.7)
    waiting = list(range(n_requests))
    requests, cancelled = {}, set()
    steps = 0
    while waiting or any(not r.finished for r in requests.values()):
        while waiting and rng.random() < 0.5:
            i = waiting.pop(0)
            requests[i] = engine.submit(prompts[i], sampling=SamplingParams(temperature=0.0),
                                        max_tokens=new_tokens[i], ignore_eos=True)
        if requests and rng.random() < 0.03:
            i = rng.choice(list(requests))
            if not requests[i].finished:
                requests[i].cancel()
                cancelled.add(i)
        engine.step()
        steps += 1
        assert steps < 5000, "the engine makes no progress"
    engine.sync()
    engine.runner.check_status()
    for i, request in requests.items():
        if i not in cancelled:
            want = plain_llama.greedy_generate(cfg, weights, prompts[i], new_tokens[i], dtype=torch.float32)
            assert list(request.output) == want, (i, request.finish_reason)
    stats = engine.cache.stats()  # everything given back: finished, cancelled and preempted alike
    assert stats["slots_used"] == 0 and all(group["used"] == 0 for group in stats["groups"])


@pytest.mark.parametrize("seed", [2, 4, 6, 8, 10, 12])
def test_seeded_sampling_does_not_depend_on_the_company(seed):
    """Temperature, top-k and top-p draws with a seed: a request gets the same tokens
    among others, in portions, preempted and recomputed, with graphs and pipelined
    steps, as when it runs alone (float32: the logits do not depend on the cutting, the
    noise is a function of seed and draw count)."""
    from pulsarlm_b200 import Engine, SamplingParams
    from pulsarlm_b200.engine.loading import load_model

    rng = random.Random(seed)
    cfg, page = rng.choice([(tiny.TINY_A, tiny.PAGE_A), (tiny.TINY_B, tiny.PAGE_B)])
    weights = tiny.random_weights(cfg, seed, torch.float32)
    with tempfile.TemporaryDirectory() as folder:
        model = load_model(tiny.write_model_dir(folder, cfg, weights), "float32", "cuda:0")
    n_requests = rng.choice([3, 5, 8])
    prompts = [tiny.random_tokens(cfg, rng.choice([1, 4, 20, 33, 70, 120]), seed * 100 + i) for i in range(n_requests)]
    new_tokens = [rng.choice([1, 3, 9, 20]) for _ in range(n_requests)]
    params = [SamplingParams(temperature=rng.choice([0.0, 0.7, 1.3]), top_k=rng.choice([0, 0, 5, 50]),
                             top_p=rng.choice([1.0, 1.0, 0.9, 0.5]), seed=rng.randrange(1 << 40))
              for _ in range(n_requests)]
    largest = max(len(p) + n for p, n in zip(prompts, new_tokens))
    alone = Engine(model, n_pages=-(-largest // page) + 2, page_size=page, max_requests=2, stop_ids=[],
                   cuda_graphs=False, lookahead=False)
    want = [alone.generate([p], s, max_tokens=n, ignore_eos=True)[0] for p, s, n in zip(prompts, params, new_tokens)]
    engine = Engine(model, n_pages=-(-largest // page) + rng.choice([0, 1, 3, 10, 40]), page_size=page,
                    prefill_tokens_per_step=rng.choice([2, 7, 32, 256]), max_requests=rng.choice([2, 4, 8]),
                    stop_ids=[], cuda_graphs=rng.random() < 0.7, lookahead=rng.random() < 0.7)
    waiting = list(range(n_requests))
    requests = {}
    steps = 0
    while waiting or any(not r.finished for r in requests.values()):
        while waiting and rng.random() < 0.5:
            i = waiting.pop(0)
            requests[i] = engine.submit(prompts[i], sampling=params[i], max_tokens=new_tokens[i], ignore_eos=True)
        engine.step()
        steps += 1
        assert steps < 5000, "the engine makes no progress"
    engine.sync()
    engine.runner.check_status()
    for i, request in requests.items():
        assert list(request.output) == want[i], (i, params[i])


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_stop_tokens_under_pipelined_steps(seed):
    """Steps pipelined one deep plan a request on as if it did not stop; one that draws a
    stop id has then run one token too many, which must leave no trace: the same tokens
    and reasons as an engine that reads every step's ids before it plans the next, under
    seeded sampling, tight pages, prompt portions beside single tokens, a cancellation,
    with and without captured steps. Everything is given back at the end."""
    from pulsarlm_b200 import Engine, SamplingParams
    from pulsarlm_b200.engine.loading import load_model

    rng = random.Random(seed)
    cfg, page = rng.choice([(tiny.TINY_A, tiny.PAGE_A), (tiny.TINY_B, tiny.PAGE_B)])
    weights = tiny.random_weights(cfg, seed, torch.float32)
    with tempfile.TemporaryDirectory() as folder:
        model = load_model(tiny.write_model_dir(folder, cfg, weights), "float32", "cuda:0")
    n_requests = 8
    prompts = [tiny.random_tokens(cfg, rng.choice([1, 4, 20, 33, 70]), seed * 100 + i) for i in range(n_requests)]
    new_tokens = [rng.choice([0, 1, 2, 9, 20]) for _ in range(n_requests)]
    params = [SamplingParams(temperature=rng.choice([0.0, 0.9]), top_k=rng.choice([0, 20]), seed=rng.randrange(1 << 40))
              for _ in range(n_requests)]
    largest = max(len(p) + n for p, n in zip(prompts, new_tokens))
    plain = Engine(model, n_pages=-(-largest // page) + 2, page_size=page, max_requests=2, stop_ids=[],
                   cuda_graphs=False, lookahead=False)
    free_run = [plain.generate([p], s, max_tokens=n, ignore_eos=True)[0] for p, s, n in zip(prompts, params, new_tokens)]
    # stop ids that some requests meet on the way (not as their last token), and some never
    stops = sorted({out[len(out) // 2] for out in free_run[::2] if len(out) >= 3})
    assert stops
    ignore = [rng.random() < 0.25 for _ in range(n_requests)]
    want = []
    for out, ignores in zip(free_run, ignore):
        cut = next((i + 1 for i, t in enumerate(out) if t in stops), len(out)) if not ignores else len(out)
        want.append((out[:cut], "stop" if cut < len(out) or (out and out[-1] in stops and not ignores) else "length"))
    engine = Engine(model, n_pages=-(-largest // page) + rng.choice([0, 2, 10]), page_size=page,
                    prefill_tokens_per_step=rng.choice([3, 16, 256]), max_requests=rng.choice([2, 4, 8]),
                    stop_ids=stops, cuda_graphs=rng.random() < 0.6, lookahead=True)
    waiting = list(range(n_requests))
    requests, cancelled = {}, None
    steps = 0
    while waiting or any(not r.finished for r in requests.values()):
        while waiting and rng.random() < 0.5:
            i = waiting.pop(0)
            requests[i] = engine.submit(prompts[i], sampling=params[i], max_tokens=new_tokens[i], ignore_eos=ignore[i])
        if cancelled is None and steps == 7 and requests:
            cancelled = rng.choice(list(requests))
            requests[cancelled].cancel()
        engine.step()
        steps += 1
        assert steps < 5000, "the engine makes no progress"
    engine.sync()
    engine.runner.check_status()
    for i, request in requests.items():
        if i == cancelled and request.finish_reason == "cancelled":
            assert list(request.output) == want[i][0][: len(request.output)]
        else:
            assert (list(request.output), request.finish_reason) == want[i], (i, stops, free_run[i])
    stats = engine.cache.stats()
    assert stats["slots_used"] == 0 and all(group["used"] == 0 for group in stats["groups"])


@pytest.mark.parametrize("seed", [1, 9, 17, 58])
def test_bfloat16_generation_with_graphs_at_tensor_core_head_sizes(seed):
    """bfloat16, head sizes 64 and 128, one to seventeen requests with prompts of up to
    900 tokens through the engine (scheduler's portions, graph-replayed and pipelined
    decode steps): bfloat16 may flip a near-tie, so the tokens are not compared; the
    logits row each token was drawn from must match the plain implementation's row
    for the generated sequence, and the token must be that row's argmax."""
    generation_against_plain(seed, random.Random(seed).choice([64, 128]))


@pytest.mark.parametrize("seed,head_dim", [(3, 96), (4, 80), (5, 32), (6, 48), (7, 112), (8, 96)])
def test_bfloat16_generation_with_graphs_at_the_other_head_sizes_of_the_mma_kernels(seed, head_dim):
    """The same at the head sizes that only the mma.sync attention kernels take (prompt
    portions on `attention_prefill`, single tokens on `attention_decode`, the rotation
    folded in where the head size is a multiple of 32)."""
    generation_against_plain(seed, head_dim)


def generation_against_plain(seed, head_dim):
    import plain_llama as plain
    from pulsarlm_b200 import Engine, SamplingParams
    from pulsarlm_b200.engine.loading import load_model

    rng = random.Random(seed)
    n_kv = rng.choice([1, 2, 4])
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": rng.choice([1, 2]),
           "hidden_size": rng.choice([256, 384]), "num_attention_heads": n_kv * rng.choice([1, 2, 3, 4, 8]),
           "num_key_value_heads": n_kv, "head_dim": head_dim, "intermediate_size": 512,
           "vocab_size": 512, "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
           "max_position_embeddings": 8192}
    weights = tiny.random_weights(cfg, seed, torch.bfloat16)
    with tempfile.TemporaryDirectory() as folder:
        model = load_model(tiny.write_model_dir(folder, cfg, weights), "bfloat16", "cuda:0")
    n_requests = rng.choice([1, 2, 5, 9, 17])
    prompts = [tiny.random_tokens(cfg, rng.choice([5, 100, 400, 900]), seed * 50 + i) for i in range(n_requests)]
    new_tokens = rng.choice([4, 12])
    page = rng.choice([16, 32])
    engine = Engine(model, n_pages=sum(len(p) + new_tokens for p in prompts) // page + n_requests + 4, page_size=page,
                    prefill_tokens_per_step=rng.choice([64, 256, 1024]), max_requests=32, stop_ids=[],
                    lookahead=rng.random() < 0.7, record_logits=True)
    requests = [engine.submit(p, sampling=SamplingParams(temperature=0.0), max_tokens=new_tokens, ignore_eos=True)
                for p in prompts]
    while any(not r.finished for r in requests):
        engine.step()
    engine.sync()
    engine.runner.check_status()
    assert engine.runner.graph_steps > 0
    from harness import TOLERANCE, record_error

    for prompt, request in zip(prompts, requests):
        output = list(request.output)
        assert len(output) == new_tokens == len(request.logits)
        assert output == [int(row.argmax()) for row in request.logits]
        reference = plain.forward(cfg, weights, list(prompt) + output[:-1], dtype=torch.float32)
        err = plain.max_relative_error(torch.stack(request.logits), reference[len(prompt) - 1:])
        record_error("bfloat16", "random configurations through the engine with graphs", err, TOLERANCE["bfloat16"])
        assert err < TOLERANCE["bfloat16"], (err, cfg)


@pytest.mark.parametrize("seed,shape", [(2, None), (7, None), (14, None), (22, None),
                                        (31, (128, 8, 1, 20)), (32, (64, 8, 2, 24)), (33, (128, 4, 4, 33))])
def test_many_requests_of_unequal_lengths_through_work_lists_and_native_layers(seed, shape):
    """bfloat16 at tensor-core head sizes, 20 to 48 requests whose prompts run from 3 to
    2,600 tokens, drawn at random: prompt portions beside single tokens (a layer from one
    native call), captured decode steps with the decode kernel's work list cut by the true
    lengths and refreshed before every replay, the rotation folded into it, pipelined or
    not. The logits every generated token was drawn from, for the longest, the shortest and
    a few other requests, against the plain implementation on the request's own prefix.
    The cases with a shape (head size, kv heads, group, requests) are so many requests that
    equal shares of their keys would split in two or three: replays with unequal lengths
    then have captures of their own that walk a work list."""
    from harness import TOLERANCE, record_error
    from pulsarlm_b200 import Engine, SamplingParams
    from pulsarlm_b200.engine.loading import load_model

    rng = random.Random(seed)
    hd, nkv, group = rng.choice([64, 128]), rng.choice([1, 2, 4, 8]), rng.choice([1, 2, 4])
    if shape is not None:
        hd, nkv, group = shape[:3]
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": rng.choice([1, 2]),
           "hidden_size": rng.choice([256, 384]), "num_attention_heads": nkv * group, "num_key_value_heads": nkv,
           "head_dim": hd, "intermediate_size": 512, "vocab_size": 512, "rope_theta": 500000.0,
           "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 8192}
    weights = tiny.random_weights(cfg, seed, torch.bfloat16)
    with tempfile.TemporaryDirectory() as folder:
        model = load_model(tiny.write_model_dir(folder, cfg, weights), "bfloat16", "cuda:0")
    n_req = rng.choice([20, 33, 48]) if shape is None else shape[3]
    lens = [rng.choice([3, 40, 200, 700, 1500, 2600]) + rng.randrange(0, 30) for _ in range(n_req)]
    prompts = [tiny.random_tokens(cfg, n, seed * 100 + i) for i, n in enumerate(lens)]
    new = rng.choice([3, 9, 20])
    page = rng.choice([16, 32, 64])
    engine = Engine(model, n_pages=sum(-(-(len(p) + new + 1) // page) for p in prompts) + 8, page_size=page,
                    # (with a shape: every prompt in the first step, so that all decode together)
                    prefill_tokens_per_step=rng.choice([256, 512, 2048]) if shape is None else 1 << 17,
                    max_requests=64, stop_ids=[], lookahead=rng.random() < 0.7, record_logits=True)
    greedy = SamplingParams(temperature=0.0)
    requests = [engine.submit(p, sampling=greedy, max_tokens=new, ignore_eos=True) for p in prompts]
    while engine.has_work():
        engine.step()
    engine.sync()
    engine.runner.check_status()
    assert engine.runner.graph_steps > 0
    if shape is not None:
        assert any(len(key) > 2 for key in engine.runner._graphs), list(engine.runner._graphs)
    order = sorted(range(n_req), key=lambda i: lens[i])
    picks = {order[0], order[-1], order[len(order) // 2]} | set(rng.sample(range(n_req), 3))
    worst = 0.0
    for i in picks:
        r = requests[i]
        assert len(r.output) == new and len(r.logits) == new
        reference = plain_llama.forward(cfg, weights, list(prompts[i]) + list(r.output), dtype=torch.float32)
        for j in range(new):
            want = reference[len(prompts[i]) - 1 + j].double()
            err = float((r.logits[j].double() - want).abs().max() / want.abs().max())
            worst = max(worst, err)
            assert err < TOLERANCE["bfloat16"], (seed, i, j, err)
    record_error("bfloat16", "many requests of unequal lengths through the engine", worst, TOLERANCE["bfloat16"])
