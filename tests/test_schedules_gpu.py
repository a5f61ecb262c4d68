"""Schedules of the product path that the small cutting tests do not reach: captured
decode steps over block tables of several widths and the hand-over between them, a
captured step padded to its size, the scheduler (portions, preemption and
recomputation, pipelined decode steps) over the tensor-core kernels in bfloat16, the
mixed schedule with recycled pages at real layer sizes, the bound on the memory that
captured steps hold, and a kernel's error reaching the caller of Engine.step. Every
comparison is of logits with the plain implementation."""

import random
import tempfile

import pytest
import torch

import plain_llama
import tiny
from harness import TOLERANCE, record_error, replay
from test_model_gpu import mixed_schedule

pytestmark = pytest.mark.gpu


def small_config(head_dim: int, n_heads: int, n_kv: int, layers: int = 2, hidden: int = 256, vocab: int = 512) -> dict:
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": layers,
            "hidden_size": hidden, "num_attention_heads": n_heads, "num_key_value_heads": n_kv, "head_dim": head_dim,
            "intermediate_size": 512, "vocab_size": vocab, "rope_theta": 500000.0,
            "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                             "original_max_position_embeddings": 1024},
            "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 8192}


def load(cfg: dict, weights: dict, dtype: str):
    from pulsarlm_b200.engine.loading import load_model

    with tempfile.TemporaryDirectory() as folder:
        return load_model(tiny.write_model_dir(folder, cfg, weights), dtype, "cuda:0")


def worst_error(rows: list, reference: torch.Tensor, positions: list) -> tuple[float, int]:
    """Largest relative error of the rows against the reference's rows at `positions`, and where."""
    got = torch.stack([r.float().cpu() for r in rows]).double()
    want = reference[positions].double()
    per_row = (got - want).abs().amax(dim=1) / want.abs().max()
    at = int(per_row.argmax())
    return float(per_row[at]), positions[at]


@pytest.mark.parametrize("head_dim,n_heads,n_kv", [(128, 4, 1), (64, 8, 2)])
def test_captured_decode_steps_across_table_widths(head_dim, n_heads, n_kv):
    """One request decodes from 1,000 to 2,150 tokens through captured steps: its block
    table outgrows two captures (64 and 128 pages wide), the split count of the decode
    attention is chosen from the capture's bound, not from the true length, and at batch
    1 it reaches the largest in-cluster split and the merge through scratch memory.
    Every step's logits are compared with the plain implementation; then the same
    request through Engine.generate (pipelined steps) must draw the same tokens."""
    from pulsarlm_b200 import Engine, SamplingParams
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.engine.runner import ModelRunner, StepEntry
    from pulsarlm_b200.parts.attention import decode_splits

    cfg = small_config(head_dim, n_heads, n_kv)
    weights = tiny.random_weights(cfg, 21, torch.bfloat16)
    model = load(cfg, weights, "bfloat16")
    prompt = tiny.random_tokens(cfg, 1000, seed=8)
    n_new = 1150
    runner = ModelRunner(model, CacheManager(model.cache_needs(), 16, 140, 2, torch.bfloat16, "cuda:0"))
    first = runner.step([StepEntry("r", prompt, [len(prompt) - 1])])
    rows = [first[0].clone()]
    tokens = [int(first[0].argmax())]
    greedy = SamplingParams(temperature=0.0)
    for i in range(n_new - 1):
        ids = runner.decode_step([StepEntry("r", [tokens[-1]], [0])], [greedy], [0], [i + 1])
        rows.append(runner.last_graph.logits[0].clone())
        tokens.append(int(ids[0]))
    runner.check_status()
    widths = sorted(width for _, width in runner._graphs)
    assert widths == [64, 128, 192], widths
    assert decode_splits(n_kv, 192 * 16, torch.device("cuda:0"), head_dim, n_heads // n_kv) >= 16
    sequence = prompt + tokens
    reference = plain_llama.forward(cfg, weights, sequence[:-1], dtype=torch.float64)
    positions = list(range(len(prompt) - 1, len(sequence) - 1))
    err, where = worst_error(rows, reference, positions)
    record_error("bfloat16", f"captured decode to 2,150 tokens, head size {head_dim}", err, TOLERANCE["bfloat16"])
    assert err < TOLERANCE["bfloat16"], (err, where)
    # every drawn token is the argmax of the row it was drawn from
    assert tokens == [int(r.argmax()) for r in rows]

    engine = Engine(model, n_pages=140, page_size=16, prefill_tokens_per_step=1024, max_requests=2, stop_ids=[])
    assert engine.generate([prompt], greedy, max_tokens=n_new, ignore_eos=True)[0] == tokens
    assert engine.runner.graph_steps >= n_new - 1 and engine.lookahead


def test_a_captured_step_padded_to_its_size_serves_fewer_entries():
    """Five, six and seven requests decode through the capture for eight: the padding rows
    write to the cache's spare page and change nothing for the others; the capture is
    made once."""
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.engine.runner import ModelRunner, StepEntry, graph_entries_bucket
    from pulsarlm_b200.sampling.params import SamplingParams

    assert [graph_entries_bucket(n) for n in (1, 3, 4, 5, 8, 9, 17, 33, 64, 65)] == [1, 3, 4, 8, 8, 12, 24, 40, 64, 80]
    cfg = small_config(64, 4, 2, layers=2)
    weights = tiny.random_weights(cfg, 5, torch.bfloat16)
    model = load(cfg, weights, "bfloat16")
    runner = ModelRunner(model, CacheManager(model.cache_needs(), 16, 64, 8, torch.bfloat16, "cuda:0"))
    prompts = {i: tiny.random_tokens(cfg, 20 + 13 * i, seed=60 + i) for i in range(7)}
    fed = {i: list(p[:-6]) for i, p in prompts.items()}
    runner.step([StepEntry(i, fed[i], []) for i in prompts])
    greedy = SamplingParams(temperature=0.0)
    rows: dict = {i: [] for i in prompts}
    for step in range(6):
        live = [i for i in prompts if i < 5 + step % 3]  # five, six, seven, five, ...
        entries = [StepEntry(i, [prompts[i][len(fed[i])]], [0]) for i in live]
        runner.decode_step(entries, [greedy] * len(live), [0] * len(live), [0] * len(live))
        for row, i in enumerate(live):
            rows[i].append((len(fed[i]), runner.last_graph.logits[row].clone()))
            fed[i].append(prompts[i][len(fed[i])])
    runner.check_status()
    assert runner.graph_captures == 1 and list(runner._graphs) == [(8, 64)]
    for i, got in rows.items():
        reference = plain_llama.forward(cfg, weights, prompts[i], dtype=torch.float64)
        err, where = worst_error([r for _, r in got], reference, [p for p, _ in got])
        assert err < TOLERANCE["bfloat16"], (i, err, where)


@pytest.mark.parametrize("seed", [2, 3, 5, 8])
def test_bfloat16_scheduler_under_page_pressure_over_the_tensor_core_kernels(seed):
    """Requests arrive at random into an engine whose pages do not hold them all: bfloat16
    at head sizes 64 and 128, prompts up to 700 tokens cut into portions (the tcgen05
    prompt kernel), captured and pipelined decode steps, the newest request preempted and
    recomputed. The engine records the logits row every kept token was drawn from; each
    is compared with the plain implementation's row for the request's own sequence."""
    from pulsarlm_b200 import Engine, SamplingParams

    rng = random.Random(seed)
    head_dim = rng.choice([64, 128])
    n_kv = rng.choice([1, 2])
    cfg = small_config(head_dim, n_kv * rng.choice([2, 3, 4]), n_kv, layers=rng.choice([1, 2]))
    weights = tiny.random_weights(cfg, seed, torch.bfloat16)
    model = load(cfg, weights, "bfloat16")
    n_requests = 6
    prompts = [tiny.random_tokens(cfg, rng.choice([30, 150, 400, 700]), seed * 40 + i) for i in range(n_requests)]
    new_tokens = [rng.choice([8, 20, 40]) for _ in range(n_requests)]
    page = 16
    needs = sorted(-(-(len(p) + n) // page) for p, n in zip(prompts, new_tokens))
    n_pages = needs[-1] + needs[-2] // 2 + 2  # the largest request and half of the next: the rest must wait or go
    engine = Engine(model, n_pages=n_pages, page_size=page, prefill_tokens_per_step=rng.choice([64, 256]),
                    max_requests=4, stop_ids=[], record_logits=True)
    assert engine.cuda_graphs and engine.lookahead
    waiting = list(range(n_requests))
    requests: dict = {}
    steps = 0
    while waiting or any(not r.finished for r in requests.values()):
        while waiting and rng.random() < 0.4:
            i = waiting.pop(0)
            requests[i] = engine.submit(prompts[i], sampling=SamplingParams(temperature=0.0),
                                        max_tokens=new_tokens[i], ignore_eos=True)
        engine.step()
        steps += 1
        assert steps < 5000, "the engine makes no progress"
    engine.sync()
    engine.runner.check_status()
    assert engine.scheduler.preemptions > 0, "the pages were meant to run out"
    assert engine.runner.graph_steps > 0
    worst = 0.0
    for i, request in requests.items():
        assert request.finish_reason == "length" and len(request.output) == new_tokens[i] == len(request.logits)
        sequence = prompts[i] + list(request.output)
        reference = plain_llama.forward(cfg, weights, sequence[:-1], dtype=torch.float64)
        positions = list(range(len(prompts[i]) - 1, len(sequence) - 1))
        err, where = worst_error(request.logits, reference, positions)
        worst = max(worst, err)
        assert err < TOLERANCE["bfloat16"], (i, err, where, request.preemptions)
        assert list(request.output) == [int(r.argmax()) for r in request.logits]
    record_error("bfloat16", f"scheduler under page pressure, head size {head_dim}", worst, TOLERANCE["bfloat16"])
    stats = engine.cache.stats()
    assert stats["slots_used"] == 0 and all(group["used"] == 0 for group in stats["groups"])


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_mixed_batches_with_page_reuse_at_real_layer_sizes(dtype):
    """Up to four live requests, portions of some beside single tokens of others, with
    room for the four longest and not a page more, at the Llama-3.1-8B layer sizes (two
    layers; a small vocabulary keeps the plain implementation quick)."""
    from pulsarlm_b200 import models  # noqa: F401
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.config.registry import read_model_config
    from pulsarlm_b200.engine.runner import ModelRunner
    from pulsarlm_b200.models.model import Model
    from pulsarlm_b200.weights.loader import check_tensors
    from test_large_gpu import CONFIG

    config = dict(CONFIG, vocab_size=2048)
    weights = tiny.random_weights(config, seed=13, dtype=torch.bfloat16)
    torch_dtype = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    device = torch.device("cuda:0")
    arch, cfg = read_model_config(config)
    model = Model(arch.describe(cfg), torch_dtype, device)
    model.load(check_tensors("test", model.tensor_needs(), weights, torch_dtype, device))
    lengths = [40, 197, 64, 33, 320, 18, 75, 150, 101, 29]
    reqs = {f"r{n}": tiny.random_tokens(config, n, seed=300 + n) for n in lengths}
    page = 16
    n_pages = sum(sorted(-(-n // page) for n in lengths)[-4:])
    runner = ModelRunner(model, CacheManager(model.cache_needs(), page, n_pages, 4, torch_dtype, device))
    got = replay(runner, mixed_schedule(reqs, random.Random(5)))
    # The requests need more pages in all than the pool has: some page served two requests.
    assert sum(-(-n // page) for n in lengths) > n_pages >= runner.cache.groups[0].pool.high_water > n_pages // 3
    assert runner.cache.free_pages() == n_pages
    worst = 0.0
    for r, rows in got.items():
        reference = plain_llama.forward(config, weights, reqs[r], dtype=torch.float32)
        positions = sorted(rows)
        err, where = worst_error([rows[p] for p in positions], reference, positions)
        worst = max(worst, err)
        assert err < TOLERANCE[dtype], (r, err, where)
    record_error(dtype, "mixed schedule with page reuse at 8B layer sizes", worst, TOLERANCE[dtype])


def test_two_engines_over_one_model_take_turns():
    """A model serves one cache at a time; engines that share its weights point its layers
    at their own cache before they step, so they can be used in turn: eager prompt steps,
    captures and replays of one engine between those of the other."""
    from pulsarlm_b200 import Engine, SamplingParams

    cfg = small_config(64, 4, 2, layers=2)
    weights = tiny.random_weights(cfg, 9, torch.bfloat16)
    model = load(cfg, weights, "bfloat16")
    prompts = [tiny.random_tokens(cfg, n, seed=70 + n) for n in (40, 150)]
    greedy = SamplingParams(temperature=0.0)
    alone = Engine(model, n_pages=40, page_size=16, max_requests=2, stop_ids=[])
    want = alone.generate(prompts, greedy, max_tokens=24, ignore_eos=True)
    first = Engine(model, n_pages=64, page_size=16, max_requests=2, stop_ids=[])
    second = Engine(model, n_pages=9, page_size=32, max_requests=2, stop_ids=[], prefill_tokens_per_step=64)
    a = [first.submit(p, sampling=greedy, max_tokens=24, ignore_eos=True) for p in prompts]
    b = [second.submit(p, sampling=greedy, max_tokens=24, ignore_eos=True) for p in prompts]
    while any(not r.finished for r in a + b):
        first.step()
        second.step()
    first.sync(), second.sync()
    first.runner.check_status(), second.runner.check_status()
    assert [list(r.output) for r in a] == want
    # the second engine cuts the prompts differently (pages of 32, portions of 64): its bfloat16 tokens
    # may differ at a near-tie, so it is held to the plain logits instead
    for request, prompt in zip(b, prompts):
        logits = plain_llama.forward(cfg, weights, prompt + list(request.output)[:-1])
        for i, token in enumerate(request.output):
            row = logits[len(prompt) - 1 + i]
            assert float((row.max() - row[token]) / row.abs().max()) <= TOLERANCE["bfloat16"]


def test_captured_steps_hold_a_bounded_amount_of_memory():
    """An engine stepped through many (entries, table width) shapes keeps at most
    `max_graphs` captures, and what the device holds stops growing once it has them."""
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.engine.runner import ModelRunner, StepEntry
    from pulsarlm_b200.sampling.params import SamplingParams

    cfg = small_config(64, 4, 2, layers=1, vocab=4096)
    model = load(cfg, tiny.random_weights(cfg, 1, torch.bfloat16), "bfloat16")
    cache = CacheManager(model.cache_needs(), 16, 40 * 184, 40, torch.bfloat16, "cuda:0")
    runner = ModelRunner(model, cache)
    runner.max_graphs = 6
    greedy = SamplingParams(temperature=0.0)
    lengths = [900, 1900, 2900]  # tables 64, 128 and 192 pages wide after one more token
    for b in range(40):
        assert cache.open(b) is not None

    def decode(batch: int, length: int) -> None:
        for b in range(batch):  # (contents do not matter: set the lengths without a prefill)
            cache.close(b)
            cache.open(b)
            cache.reserve(b, length)
            cache.commit(b, length)
        entries = [StepEntry(b, [1 + b], [0]) for b in range(batch)]
        runner.decode_step(entries, [greedy] * batch, [0] * batch, [0] * batch)

    shapes = [(batch, length) for batch in (1, 2, 3, 4, 7, 11, 16, 23, 31, 40) for length in lengths]
    for batch, length in shapes[:12]:
        decode(batch, length)
    torch.cuda.synchronize()
    assert len(runner._graphs) == 6
    reserved = torch.cuda.memory_reserved()
    for batch, length in shapes[12:] + shapes:
        decode(batch, length)
    torch.cuda.synchronize()
    runner.check_status()
    assert len(runner._graphs) == 6 and runner.graph_captures >= len(shapes)
    # logits of the largest shape: 40 x 4,096 floats; the pool may grow by a few such buffers, not by 48 captures
    assert torch.cuda.memory_reserved() - reserved < 64 << 20


def test_a_kernels_error_reaches_the_caller_of_step():
    """A block-table row that names no page makes the kernels flag the step; the flag
    travels with the sampled ids and Engine.step raises, in the eager path and in the
    captured one."""
    from pulsarlm_b200 import Engine, SamplingParams

    cfg = small_config(64, 4, 2, layers=1)
    model = load(cfg, tiny.random_weights(cfg, 2, torch.bfloat16), "bfloat16")
    for graphs in (False, True):
        engine = Engine(model, n_pages=16, page_size=16, max_requests=2, stop_ids=[], cuda_graphs=graphs)
        request = engine.submit(tiny.random_tokens(cfg, 20, seed=1), sampling=SamplingParams(temperature=0.0),
                                max_tokens=40, ignore_eos=True)
        for _ in range(4):
            engine.step()
        engine.sync()
        assert len(request.output) >= 2
        # Break the book-keeping behind the engine's back: the request's pages go to
        # nobody, so its next table row is empty.
        fill = engine.cache.fill_tables

        def broken(group, handles, table, slots):
            longest = fill(group, handles, table, slots)
            table[...] = -1
            return longest

        engine.cache.fill_tables = broken
        engine.cache.table_rows = lambda group, requests, width_multiple=8: \
            -torch.ones((len(requests), 8), dtype=torch.int32).numpy()
        with pytest.raises(RuntimeError, match="block-table entry"):
            for _ in range(3):
                engine.step()
            engine.sync()
        torch.cuda.synchronize()
