"""Configurations drawn at random (head sizes in steps of 16 from 16 to 128, any number
of heads and groups, widths and vocabularies that are no powers of two, one to four
layers, either RoPE form, tied or not) through the engine's step function, cut three
ways, against the plain implementation, in float32 and in bfloat16. The drawn sizes
reach every attention kernel: tensor-core kernels at head sizes 64 and 128 with even
and odd groups, the CUDA-core kernel elsewhere."""

import random
import tempfile

import pytest
import torch

import plain_llama
import tiny
from harness import TOLERANCE, replay

pytestmark = pytest.mark.gpu


def draw_config(rng: random.Random) -> dict:
    n_kv = rng.choice([1, 2, 3, 4])
    cfg = {
        "architectures": ["LlamaForCausalLM"],
        "model_type": "llama",
        "num_hidden_layers": rng.choice([1, 2, 3, 4]),
        "hidden_size": rng.choice([40, 64, 72, 96, 136, 200, 264]),
        "num_attention_heads": n_kv * rng.choice([1, 2, 3, 4, 5, 8]),
        "num_key_value_heads": n_kv,
        "head_dim": rng.choice([16, 32, 48, 64, 80, 96, 112, 128]),
        "intermediate_size": rng.choice([48, 100, 172, 256, 344]),
        "vocab_size": rng.choice([97, 256, 1000, 1531]),
        "rope_theta": rng.choice([10000.0, 500000.0, 1e6]),
        "rms_norm_eps": rng.choice([1e-5, 1e-6, 3e-4]),
        "tie_word_embeddings": rng.choice([True, False]),
        "max_position_embeddings": 2048,
    }
    if rng.random() < 0.5:
        cfg["rope_scaling"] = {"rope_type": "llama3", "factor": rng.choice([2.0, 8.0, 32.0]), "low_freq_factor": 1.0,
                               "high_freq_factor": rng.choice([2.0, 4.0]),
                               "original_max_position_embeddings": rng.choice([32, 64, 256])}
    return cfg


def draw_schedules(rng: random.Random, requests: dict) -> dict:
    """Each request whole; each in portions of changing size; and two waves of requests
    that advance together by random amounts, the second wave on the first one's pages."""
    whole = [([(r, t, [0, len(t) - 1])], [r]) for r, t in requests.items()]
    portions = []
    for r, t in requests.items():
        at = 0
        while at < len(t):
            n = min(len(t) - at, rng.choice([1, 2, 2, 3, 5, 13, 31, 64, 130]))
            portions.append(([(r, t[at : at + n], [n - 1])], [r] if at + n >= len(t) else []))
            at += n
    names = list(requests)
    half = (len(names) + 1) // 2
    fed = {r: 0 for r in names}
    mixed = []
    for wave in (names[:half], names[half:]):
        live = list(wave)
        while live:
            entries, ends = [], []
            for r in list(live):
                if rng.random() < 0.2 and len(live) > 1:
                    continue  # left out of this step
                t = requests[r]
                n = min(len(t) - fed[r], rng.choice([1, 1, 1, 2, 4, 9, 40]))
                entries.append((r, t[fed[r] : fed[r] + n], [n - 1] if rng.random() < 0.8 else []))
                fed[r] += n
                if fed[r] >= len(t):
                    ends.append(r)
                    live.remove(r)
            if entries:
                mixed.append((entries, ends))
    return {"whole": whole, "portions": portions, "mixed": mixed}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [3, 5, 9, 103, 106, 111])
def test_a_configuration_drawn_at_random(seed, dtype):
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.engine.loading import load_model
    from pulsarlm_b200.engine.runner import ModelRunner

    rng = random.Random(seed)
    cfg = draw_config(rng)
    torch_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
    weights = tiny.random_weights(cfg, seed, torch_dtype)
    lengths = [rng.choice([3, 17, 64, 65, 150, 300]) for _ in range(rng.choice([2, 3, 4]))]
    requests = {f"r{i}": tiny.random_tokens(cfg, n, 10 * seed + i) for i, n in enumerate(lengths)}
    plain = {r: plain_llama.forward(cfg, weights, t) for r, t in requests.items()}
    page = rng.choice([16, 32])
    names = list(requests)
    half = (len(names) + 1) // 2
    # pages for the larger wave only (each request's length rounded up to 64): the second wave reuses them
    room = max(sum(-(-len(requests[r]) // 64) * 64 for r in wave) for wave in (names[:half], names[half:]) if wave)
    with tempfile.TemporaryDirectory() as folder:
        model = load_model(tiny.write_model_dir(folder, cfg, weights), dtype, "cuda:0")
    for name, steps in draw_schedules(rng, requests).items():
        runner = ModelRunner(model, CacheManager(model.cache_needs(), page, room // page, 4, torch_dtype, "cuda:0"))
        got = replay(runner, steps)
        assert set(got) == set(requests) and all(len(rows) >= 1 for rows in got.values())
        for r, rows in got.items():
            positions = sorted(rows)
            err = plain_llama.max_relative_error(torch.stack([rows[p] for p in positions]), plain[r][positions])
            assert err < TOLERANCE[dtype], (name, r, err, cfg)


@pytest.mark.parametrize("seed", [0, 3, 5, 11, 12, 23])
def test_longer_prompts_reach_the_tensor_core_attention_paths(seed):
    """bfloat16 at head sizes 64 and 128 with histories of up to 1,500 tokens, three
    requests advancing together in portions of 1 to 600 tokens: short portions after
    long histories (keys split over CTAs and merged), portions longer than one tile
    with odd groups (tiles of 256 rows), single tokens over many keys (splits merged
    in a cluster), pages of 16, 32 or 64 tokens."""
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.engine.loading import load_model
    from pulsarlm_b200.engine.runner import ModelRunner

    rng = random.Random(seed)
    n_kv = rng.choice([1, 2, 4])
    cfg = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": rng.choice([1, 2]),
        "hidden_size": rng.choice([256, 384, 520]), "num_attention_heads": n_kv * rng.choice([1, 2, 3, 4, 8]),
        "num_key_value_heads": n_kv, "head_dim": rng.choice([64, 128]), "intermediate_size": rng.choice([512, 1000]),
        "vocab_size": 512, "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
        "max_position_embeddings": 8192,
    }
    weights = tiny.random_weights(cfg, seed, torch.bfloat16)
    with tempfile.TemporaryDirectory() as folder:
        model = load_model(tiny.write_model_dir(folder, cfg, weights), "bfloat16", "cuda:0")
    lengths = [rng.choice([700, 1100, 1500]), rng.choice([300, 900]), rng.choice([40, 200])]
    requests = {f"r{i}": tiny.random_tokens(cfg, n, 7 * seed + i) for i, n in enumerate(lengths)}
    plain = {r: plain_llama.forward(cfg, weights, t, dtype=torch.float32) for r, t in requests.items()}
    fed = {r: 0 for r in requests}
    live = list(requests)
    steps = []
    while live:
        entries, ends = [], []
        for r in list(live):
            t = requests[r]
            n = min(len(t) - fed[r], rng.choice([1, 1, 2, 13, 100, 129, 256, 300, 600]))
            entries.append((r, t[fed[r] : fed[r] + n], sorted(set(rng.sample(range(n), min(n, 2)) + [n - 1]))))
            fed[r] += n
            if fed[r] >= len(t):
                ends.append(r)
                live.remove(r)
        steps.append((entries, ends))
    page = rng.choice([16, 32, 64])
    cache = CacheManager(model.cache_needs(), page, sum(lengths) // page + 8, 4, torch.bfloat16, "cuda:0")
    got = replay(ModelRunner(model, cache), steps)
    for r, rows in got.items():
        positions = sorted(rows)
        err = plain_llama.max_relative_error(torch.stack([rows[p] for p in positions]), plain[r][positions])
        assert err < TOLERANCE["bfloat16"], (r, err, cfg)
