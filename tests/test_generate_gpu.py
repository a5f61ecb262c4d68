"""Generation through the Python entry point and the command line."""

import json
import os
import subprocess
import sys

import pytest
import torch

import plain_llama
import tiny
from harness import TinyModel

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("key", ["A", "B"])
@pytest.mark.parametrize("graphs", [True, False])
def test_greedy_generation_matches_the_plain_implementation(key, graphs):
    from pulsarlm_b200 import Engine, SamplingParams

    tm = TinyModel(key, "float32")
    engine = Engine(tm.folder, dtype="float32", n_pages=24, page_size=tm.page, max_requests=4,
                    prefill_tokens_per_step=13, cuda_graphs=graphs)
    prompts = [tiny.random_tokens(tm.cfg, n, seed=n) for n in (5, 17, 33)]
    got = engine.generate(prompts, SamplingParams(temperature=0.0), max_tokens=8, ignore_eos=True)
    for prompt, tokens in zip(prompts, got):
        assert tokens == plain_llama.greedy_generate(tm.cfg, tm.weights, prompt, 8)
    assert engine.cache.free_pages() == 24
    assert (engine.runner.graph_steps > 0) == graphs


def test_greedy_generation_in_bfloat16_follows_the_plain_logits():
    """bfloat16 may flip a near-tie, so the tokens themselves are not compared: the
    engine keeps the logits row each token was drawn from, every token must be that
    row's argmax, and every row must match the plain implementation's row for the
    sequence that was generated."""
    from harness import TOLERANCE, record_error
    from pulsarlm_b200 import Engine

    tm = TinyModel("C", "bfloat16")
    engine = Engine(tm.folder, dtype="bfloat16", n_pages=32, page_size=tm.page, max_requests=4, record_logits=True)
    prompt = tiny.random_tokens(tm.cfg, 40, seed=3)
    request = engine.submit(prompt, max_tokens=12, ignore_eos=True)
    while not request.finished:
        engine.step()
    engine.sync()
    assert engine.runner.graph_steps > 0 and len(request.logits) == 12 == len(request.output)
    assert list(request.output) == [int(row.argmax()) for row in request.logits]
    reference = plain_llama.forward(tm.cfg, tm.weights, prompt + list(request.output)[:-1])
    err = plain_llama.max_relative_error(torch.stack(request.logits), reference[len(prompt) - 1:])
    record_error("bfloat16", "greedy generation through the entry point", err, TOLERANCE["bfloat16"])
    assert err < TOLERANCE["bfloat16"]


def test_temperature_sampling_is_seeded_and_chunking_does_not_change_it():
    from pulsarlm_b200 import Engine, SamplingParams

    tm = TinyModel("B", "float32")
    prompts = [tiny.random_tokens(tm.cfg, n, seed=n) for n in (1, 7, 64, 100, 200)]
    sampling = SamplingParams(temperature=0.7, seed=1234)

    def run(budget, pages, graphs=True):
        engine = Engine(tm.folder, dtype="float32", n_pages=pages, page_size=tm.page, max_requests=4,
                        prefill_tokens_per_step=budget, cuda_graphs=graphs)
        return engine.generate(prompts, sampling, max_tokens=10, ignore_eos=True), engine

    base, _ = run(13, 64)
    again, _ = run(13, 64)
    assert base == again
    other_cut, _ = run(256, 64, graphs=False)
    assert base == other_cut  # float32 logits are cut-invariant bit for bit, so the draws are too
    # 10 pages of 32 tokens cannot hold 140 + 240 tokens: the younger request is
    # preempted and recomputed, and still draws the same tokens.
    two = [prompts[3], prompts[4]]
    roomy = Engine(tm.folder, dtype="float32", n_pages=64, page_size=tm.page, prefill_tokens_per_step=13)
    tight = Engine(tm.folder, dtype="float32", n_pages=10, page_size=tm.page, prefill_tokens_per_step=13)
    want = roomy.generate(two, sampling, max_tokens=40, ignore_eos=True)
    assert tight.generate(two, sampling, max_tokens=40, ignore_eos=True) == want
    assert tight.scheduler.preemptions > 0 and roomy.scheduler.preemptions == 0
    assert want[0][:10] == base[3] and want[1][:10] == base[4]
    different, _ = Engine(tm.folder, dtype="float32", n_pages=64, page_size=tm.page).generate(
        prompts, SamplingParams(temperature=0.7, seed=99), max_tokens=10, ignore_eos=True), None
    assert different != base


def test_stop_ids_max_tokens_and_complete():
    from pulsarlm_b200 import Engine, SamplingParams, complete

    tm = TinyModel("A", "float32")
    prompt = tiny.random_tokens(tm.cfg, 9, seed=1)
    free_run = plain_llama.greedy_generate(tm.cfg, tm.weights, prompt, 8)
    engine = Engine(tm.folder, dtype="float32", n_pages=8, page_size=tm.page, stop_ids=[free_run[3]])
    stop_at = free_run.index(free_run[3])
    assert engine.generate([prompt], max_tokens=8)[0] == free_run[: stop_at + 1]
    assert engine.generate([prompt], max_tokens=8, ignore_eos=True)[0] == free_run
    assert engine.generate([prompt], max_tokens=0)[0] == []
    # complete() stops at the stop id like generate(), or at its own limit if that comes first
    assert list(complete(engine, prompt, sampling=SamplingParams(), max_tokens=3)) == free_run[: min(3, stop_at + 1)]
    assert list(complete(engine, prompt, sampling=SamplingParams(), max_tokens=8)) == free_run[: stop_at + 1]
    with pytest.raises(ValueError):
        engine.submit([tm.cfg["vocab_size"]])
    with pytest.raises(ValueError):
        engine.submit([])
    with pytest.raises(MemoryError):
        engine.generate([tiny.random_tokens(tm.cfg, 200, seed=2)], max_tokens=1)


def test_pipelined_decode_steps_change_nothing_but_the_timing():
    """With decode steps pipelined one deep (the next step is launched on the ids the
    GPU is still sampling) the tokens, the finish reasons and the freed pages are those
    of the unpipelined engine: requests that end on a stop token in mid-flight (their
    extra token is dropped), at their token limit, with different limits, sampled with
    a temperature, and with a request that arrives while the others decode."""
    from pulsarlm_b200 import Engine, SamplingParams

    tm = TinyModel("B", "float32")
    prompts = [tiny.random_tokens(tm.cfg, n, seed=10 + n) for n in (3, 20, 41, 70)]
    greedy = [plain_llama.greedy_generate(tm.cfg, tm.weights, p, 14) for p in prompts]
    stops = [greedy[1][5], greedy[2][9]]  # requests 1 and 2 stop in the middle of the others' decoding

    def run(lookahead):
        engine = Engine(tm.folder, dtype="float32", n_pages=40, page_size=tm.page, max_requests=6,
                        prefill_tokens_per_step=32, stop_ids=stops, lookahead=lookahead)
        limits = [14, 14, 14, 6]
        requests = [engine.submit(p, sampling=SamplingParams(temperature=0.0), max_tokens=m)
                    for p, m in zip(prompts, limits)]
        late = None
        calls = 0
        while any(not r.finished for r in requests) or late is None or not late.finished:
            engine.step()
            calls += 1
            if calls == 6:  # arrives while the others decode
                late = engine.submit(tiny.random_tokens(tm.cfg, 25, seed=99),
                                     sampling=SamplingParams(temperature=0.8, seed=7), max_tokens=9, ignore_eos=True)
        engine.sync()
        engine.runner.check_status()
        assert engine.cache.free_pages() == 40
        assert engine.runner.graph_steps > 0
        return [(list(r.output), r.finish_reason) for r in requests + [late]]

    piped, plain = run(True), run(False)
    assert piped == plain
    for (tokens, reason), want in zip(plain[:4], greedy):
        assert tokens == want[: len(tokens)]
    assert plain[1][1] == "stop" and plain[3][1] == "length" and len(plain[3][0]) == 6


def test_cancelling_a_request_while_its_step_is_in_flight():
    """A request cancelled between two calls of step() (its decode step already
    launched, the next not yet) ends as cancelled, keeps the tokens it had been given,
    gives its pages back, and the others go on unharmed."""
    from pulsarlm_b200 import Engine, SamplingParams

    tm = TinyModel("A", "float32")
    engine = Engine(tm.folder, dtype="float32", n_pages=24, page_size=tm.page, max_requests=4)
    prompts = [tiny.random_tokens(tm.cfg, n, seed=30 + n) for n in (6, 11)]
    keep, drop = (engine.submit(p, sampling=SamplingParams(temperature=0.0), max_tokens=12, ignore_eos=True)
                  for p in prompts)
    for _ in range(6):
        engine.step()
    assert engine._inflight is not None  # decode steps are pipelined by now
    seen = len(drop.output)
    drop.cancel()
    while not keep.finished:
        engine.step()
    engine.sync()
    assert drop.finished and drop.finish_reason == "cancelled" and seen <= len(drop.output) <= seen + 1
    assert keep.output == plain_llama.greedy_generate(tm.cfg, tm.weights, prompts[0], 12)
    assert drop.output == plain_llama.greedy_generate(tm.cfg, tm.weights, prompts[1], 12)[: len(drop.output)]
    assert engine.cache.free_pages() == 24


def test_command_line_generate_and_random_model(tmp_path):
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(tiny.TINY_A))
    env = dict(os.environ, PYTHONPATH=ROOT)
    out = subprocess.run([sys.executable, "-m", "pulsarlm_b200", "models", "random", str(tmp_path / "m"), "--config",
                          str(cfg_path), "--seed", "3", "--dtype", "float32"], env=env, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    out = subprocess.run([sys.executable, "-m", "pulsarlm_b200", "generate", str(tmp_path / "m"), "--dtype", "float32",
                          "--prompt_ids", "1,2,3,4", "--max_tokens", "5", "--kv_cache_gib", "0.01", "--ignore_eos"],
                         env=env, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    record = json.loads(out.stdout.strip().splitlines()[-1])
    assert record["prompt_ids"] == [1, 2, 3, 4] and len(record["output_ids"]) == 5

    from pulsarlm_b200 import Engine

    engine = Engine(str(tmp_path / "m"), dtype="float32", n_pages=8)
    assert engine.generate([[1, 2, 3, 4]], max_tokens=5, ignore_eos=True)[0] == record["output_ids"]


def test_a_folder_that_does_not_fit_fails_with_one_clear_error(tmp_path):
    from pulsarlm_b200 import Engine
    from pulsarlm_b200.weights.loader import WeightsError

    w = tiny.random_weights(tiny.TINY_A, 1)
    del w["model.layers.0.mlp.down_proj.weight"]
    w["extra.weight"] = torch.zeros(3)
    tiny.write_model_dir(str(tmp_path), tiny.TINY_A, w)
    with pytest.raises(WeightsError) as error:
        Engine(str(tmp_path), dtype="bfloat16", n_pages=4)
    assert "down_proj" in str(error.value) and "extra.weight" in str(error.value)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_random_weights_are_the_same_bits_on_the_host_and_on_the_device(dtype):
    """A model drawn on the device for a measurement is the model that a random model
    folder holds for the same configuration and seed."""
    from pulsarlm_b200.weights.random_init import fill_random

    for name, n, scale, offset in (("a.weight", 1000003, 0.02, 0.0), ("norm", 4097, 0.02, 1.0), ("b", 1, 3.0, 0.0)):
        host = fill_random(torch.empty(n, dtype=dtype), 11, name, scale, offset)
        device = fill_random(torch.empty(n, dtype=dtype, device="cuda:0"), 11, name, scale, offset)
        assert torch.equal(host, device.cpu()), name


def test_a_model_drawn_on_the_device_matches_the_plain_implementation_of_its_folder(tmp_path):
    """Engine(config, seed) draws weights on the device; write_random_model writes the same
    weights to a folder on the CPU; the plain implementation run on the folder's tensors
    predicts the engine's logits."""
    from harness import assert_matches_plain  # noqa: F401  (the harness' bar)
    from pulsarlm_b200 import Engine, SamplingParams
    from pulsarlm_b200.weights.random_init import write_random_model
    from pulsarlm_b200.weights.safetensors_io import SafetensorsFile

    folder = write_random_model(str(tmp_path / "m"), tiny.TINY_B, seed=9, dtype=torch.float32)
    file = SafetensorsFile(folder + "/model.safetensors")
    weights = {name: file.tensor(name).clone() for name in file.names()}
    file.close()
    engine = Engine(tiny.TINY_B, dtype="float32", device="cuda:0", n_pages=32, page_size=tiny.PAGE_B, max_requests=2,
                    seed=9)
    prompt = tiny.random_tokens(tiny.TINY_B, 23, seed=2)
    got = engine.generate([prompt], SamplingParams(temperature=0.0), max_tokens=5, ignore_eos=True)[0]
    assert got == plain_llama.greedy_generate(tiny.TINY_B, weights, prompt, 5)
