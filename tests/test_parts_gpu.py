"""Each part of a layer alone against the plain implementation, at its own sizes,
and models put together from parts in ways Llama does not use: a layer that runs
twice, a layer that reads another layer's cache, a windowed layer beside full
ones."""

import copy
import math

import pytest
import torch

import plain_llama
import tiny

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def ctx(dtype):
    from pulsarlm_b200.parts.registry import BuildContext

    return BuildContext(dtype=dtype, device=DEV)


def rel(got, want):
    return plain_llama.max_relative_error(got.cpu(), want.cpu())


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2)])
def test_norm_part(dtype, tol):
    from pulsarlm_b200.parts.registry import build_part
    from pulsarlm_b200.parts.spec import PartSpec

    norm = build_part("norm", PartSpec("rmsnorm", {"hidden_size": 100, "eps": 1e-3}, {"weight": "w"}), ctx(dtype))
    w = 1 + 0.2 * torch.randn(100)
    norm.load({"w": w.to(DEV, dtype)})
    x = torch.randn(7, 100, device=DEV)
    delta = torch.randn(7, 100, device=DEV).to(dtype)
    want = plain_llama.rms_norm((x + delta.float()).double().cpu(), w.to(dtype).double(), 1e-3)
    got = norm.forward(x, delta)
    assert rel(got, want) < tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_feed_forward_part(dtype, tol):
    from pulsarlm_b200.parts.registry import build_part
    from pulsarlm_b200.parts.spec import PartSpec

    spec = PartSpec("gated_mlp", {"hidden_size": 72, "intermediate_size": 172, "activation": "silu"},
                    {"gate": "g", "up": "u", "down": "d"})
    ff = build_part("feed_forward", spec, ctx(dtype))
    w = {"g": torch.randn(172, 72) / 8, "u": torch.randn(172, 72) / 8, "d": torch.randn(72, 172) / 13}
    w = {k: v.to(dtype) for k, v in w.items()}
    ff.load({k: v.to(DEV) for k, v in w.items()})
    h = torch.randn(11, 72).to(dtype)
    want = plain_llama.swiglu_mlp(h.double(), w["g"].double(), w["u"].double(), w["d"].double())
    assert rel(ff.forward(h.to(DEV), None), want) < tol
    with pytest.raises(ValueError):
        bad = copy.deepcopy(spec)
        bad.params["activation"] = "gelu"
        build_part("feed_forward", bad, ctx(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts(dtype):
    from pulsarlm_b200.parts.registry import build_part
    from pulsarlm_b200.parts.spec import PartSpec

    sizes = {"vocab_size": 333, "hidden_size": 40}
    emb = build_part("embedding", PartSpec("table", sizes, {"weight": "e"}), ctx(dtype))
    table = torch.randn(333, 40).to(dtype)
    emb.load({"e": table.to(DEV)})
    tokens = torch.tensor([0, 332, 17], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(tokens).cpu(), table[tokens.cpu().long()].float())
    head = build_part("head", PartSpec("linear", sizes, {"weight": None}), ctx(dtype))
    assert head.tied and head.tensor_needs(head.spec) == {}
    head.tie(emb.weight)
    h = torch.randn(5, 40).to(dtype)
    logits = head.forward(h.to(DEV))
    assert logits.dtype == torch.float32
    assert rel(logits, h.double() @ table.double().T) < (1e-5 if dtype == torch.float32 else 1e-2)


def test_position_part_matches_reference_table():
    from pulsarlm_b200.parts.registry import build_part
    from pulsarlm_b200.parts.spec import PartSpec

    llama3 = {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
              "original_max_position_embeddings": 8192.0}
    rope = build_part("position", PartSpec("rope", {"theta": 500000.0, "head_dim": 128, "rotary_dim": 128,
                                                    "llama3": llama3}), ctx(torch.float32))
    inv_freq, rotary = rope.table()
    want = plain_llama.rope_inverse_frequency(500000.0, 128, {"factor": 8.0, "low": 1.0, "high": 4.0,
                                                             "original": 8192.0})
    assert rotary == 128 and torch.allclose(inv_freq.cpu(), want, rtol=1e-14, atol=0)
    none = build_part("position", PartSpec("none"), ctx(torch.float32))
    assert none.table() == (None, 0)


# ------------------------------------------------------------------ models from parts, not Llama's layout

def run_whole(spec, weights, dtype, tokens, page=16):
    """Runs one whole request through a Model built from `spec`; returns logits."""
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.engine.runner import ModelRunner, StepEntry
    from pulsarlm_b200.models.model import Model
    from pulsarlm_b200.weights.loader import check_tensors

    model = Model(spec, dtype, DEV)
    model.load(check_tensors("test", model.tensor_needs(), weights, dtype, DEV))
    cache = CacheManager(model.cache_needs(), page, 32, 2, dtype, DEV)
    runner = ModelRunner(model, cache)
    cut = len(tokens) // 2 + 1
    first = runner.step([StepEntry("r", tokens[:cut], list(range(cut)))])
    rest = [runner.step([StepEntry("r", [t], [0])]) for t in tokens[cut:]]
    runner.check_status()
    return torch.cat([first, *rest]).cpu(), runner


def plain_variant(cfg, w, tokens, order, windows=None, cache_from=None):
    """The plain implementation's layer loop with a custom order, windows and shared caches."""
    w = {k: v.double() for k, v in w.items()}
    tokens_t = torch.tensor(tokens)
    positions = torch.arange(len(tokens))
    eps = cfg["rms_norm_eps"]
    x = plain_llama.embed(w["model.embed_tokens.weight"], tokens_t)
    for layer in order:
        p = f"model.layers.{layer}."
        h = plain_llama.rms_norm(x, w[p + "input_layernorm.weight"], eps)
        wl = dict(w)
        src = (cache_from or {}).get(layer)
        if src is not None:  # k, v come from the source layer's projections of ITS input: emulate by reuse
            raise NotImplementedError
        x = x + plain_llama.attention_block(h, wl, p, cfg, positions, (windows or {}).get(layer))
        h = plain_llama.rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + plain_llama.swiglu_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                       w[p + "mlp.down_proj.weight"])
    head = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    return plain_llama.rms_norm(x, w["model.norm.weight"], eps) @ head.T


def llama_spec(cfg):
    from pulsarlm_b200 import models  # noqa: F401
    from pulsarlm_b200.config.registry import read_model_config

    arch, typed = read_model_config(cfg)
    return arch.describe(typed)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_a_layer_named_twice_in_the_order(dtype, tol):
    cfg = tiny.TINY_B
    w = tiny.random_weights(cfg, 4, dtype)
    spec = llama_spec(cfg)
    spec.order = [0, 1, 1, 2, 0]
    tokens = tiny.random_tokens(cfg, 40, 8)
    # A layer that runs twice writes its keys twice at the same places: the second
    # pass overwrites the first pass's keys, and every query of the second pass
    # reads second-pass keys only when the whole request is one step. Cut into
    # steps, earlier positions hold second-pass keys during the first pass of a
    # later step, so here the request runs whole.
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.engine.runner import ModelRunner, StepEntry
    from pulsarlm_b200.models.model import Model
    from pulsarlm_b200.weights.loader import check_tensors

    model = Model(spec, dtype, DEV)
    model.load(check_tensors("test", model.tensor_needs(), w, dtype, DEV))
    runner = ModelRunner(model, CacheManager(model.cache_needs(), 32, 8, 2, dtype, DEV))
    got = runner.step([StepEntry("r", tokens, list(range(40)))]).cpu()
    want = plain_variant(cfg, w, tokens, spec.order)
    assert plain_llama.max_relative_error(got, want) < tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_windowed_layers_beside_full_ones(dtype, tol):
    cfg = tiny.TINY_C
    w = tiny.random_weights(cfg, 5, dtype)
    spec = llama_spec(cfg)
    spec.layers[1].mixer.params["window"] = 24
    tokens = tiny.random_tokens(cfg, 90, 2)
    got, runner = run_whole(spec, w, dtype, tokens)
    want = plain_variant(cfg, w, tokens, spec.order, windows={1: 24})
    assert plain_llama.max_relative_error(got, want) < tol
    # two groups, and the windowed one gave pages back as the request grew
    assert len(runner.cache.groups) == 2
    held = [len(runner.cache.held_pages("r", g.index)) for g in runner.cache.groups]
    assert held[0] == -(-90 // 16) and held[1] <= 24 // 16 + 2


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_a_layer_reading_another_layers_cache(dtype, tol):
    """Layer 1 has no k and v projections and attends over layer 0's keys and values."""
    cfg = tiny.TINY_A
    w = tiny.random_weights(cfg, 6, dtype)
    spec = llama_spec(cfg)
    spec.layers[1].mixer.params["cache_from"] = 0
    del w["model.layers.1.self_attn.k_proj.weight"], w["model.layers.1.self_attn.v_proj.weight"]
    tokens = tiny.random_tokens(cfg, 37, 3)
    got, runner = run_whole(spec, w, dtype, tokens)
    assert len(runner.cache.groups) == 1 and runner.cache.groups[0].layers == [0]

    # plain: layer 1's attention uses layer 0's rotated k and its v
    wd = {k: v.double() for k, v in w.items()}
    n, nh, hd = len(tokens), 4, 16
    pos = torch.arange(n)
    inv = plain_llama.rope_inverse_frequency(10000.0, hd, None)
    eps = cfg["rms_norm_eps"]
    x = plain_llama.embed(wd["model.embed_tokens.weight"], torch.tensor(tokens))
    h0 = plain_llama.rms_norm(x, wd["model.layers.0.input_layernorm.weight"], eps)
    k0 = plain_llama.rope_rotate((h0 @ wd["model.layers.0.self_attn.k_proj.weight"].T).view(n, nh, hd), pos, inv)
    v0 = (h0 @ wd["model.layers.0.self_attn.v_proj.weight"].T).view(n, nh, hd)
    for layer in (0, 1):
        p = f"model.layers.{layer}."
        h = plain_llama.rms_norm(x, wd[p + "input_layernorm.weight"], eps)
        q = plain_llama.rope_rotate((h @ wd[p + "self_attn.q_proj.weight"].T).view(n, nh, hd), pos, inv)
        o = plain_llama.causal_attention(q, k0, v0, 1 / math.sqrt(hd)).reshape(n, nh * hd)
        x = x + o @ wd[p + "self_attn.o_proj.weight"].T
        h = plain_llama.rms_norm(x, wd[p + "post_attention_layernorm.weight"], eps)
        x = x + plain_llama.swiglu_mlp(h, wd[p + "mlp.gate_proj.weight"], wd[p + "mlp.up_proj.weight"],
                                       wd[p + "mlp.down_proj.weight"])
    want = plain_llama.rms_norm(x, wd["model.norm.weight"], eps) @ wd["model.embed_tokens.weight"].T
    assert plain_llama.max_relative_error(got, want) < tol


@pytest.mark.parametrize("seed", [3, 5, 7, 9])
def test_windows_at_tensor_core_head_sizes_with_long_histories(seed):
    """bfloat16, head sizes 64 and 128: layers with windows of 17 to 700 keys beside full
    ones, two requests of up to 1,300 tokens advancing in portions of 1 to 600 tokens. The
    windowed groups give pages back as the requests grow; a kernel that read one would
    raise the status flag, which the replay checks."""
    import random

    from harness import TOLERANCE, replay
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.engine.runner import ModelRunner
    from pulsarlm_b200.models.model import Model
    from pulsarlm_b200.weights.loader import check_tensors

    rng = random.Random(seed)
    n_kv = rng.choice([1, 2])
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2,
           "hidden_size": rng.choice([128, 256]), "num_attention_heads": n_kv * rng.choice([1, 2, 3, 4]),
           "num_key_value_heads": n_kv, "head_dim": rng.choice([64, 128]), "intermediate_size": 256,
           "vocab_size": 300, "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
           "max_position_embeddings": 8192}
    w = tiny.random_weights(cfg, seed, torch.bfloat16)
    spec = llama_spec(cfg)
    windows = {rng.choice([0, 1]): rng.choice([17, 64, 100, 129, 300, 700])}
    if rng.random() < 0.5:
        windows[1 - list(windows)[0]] = rng.choice([33, 250])
    for layer, window in windows.items():
        spec.layers[layer].mixer.params["window"] = window
    model = Model(spec, torch.bfloat16, DEV)
    model.load(check_tensors("test", model.tensor_needs(), w, torch.bfloat16, DEV))
    lengths = [rng.choice([400, 900, 1300]), rng.choice([60, 500])]
    requests = {f"r{i}": tiny.random_tokens(cfg, n, 7 * seed + i) for i, n in enumerate(lengths)}
    want = {r: plain_variant(cfg, w, t, spec.order, windows=windows) for r, t in requests.items()}
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
    page = rng.choice([16, 32])
    cache = CacheManager(model.cache_needs(), page, sum(lengths) // page + 8, 4, torch.bfloat16, DEV)
    got = replay(ModelRunner(model, cache), steps)
    for r, rows in got.items():
        positions = sorted(rows)
        err = plain_llama.max_relative_error(torch.stack([rows[p] for p in positions]), want[r][positions])
        assert err < TOLERANCE["bfloat16"], (r, err, cfg, windows)


@pytest.mark.parametrize("seed", [1, 4, 6])
def test_windowed_groups_with_pools_of_their_own_size_through_the_engine(seed):
    """A windowed layer beside a full one through `Engine` (scheduler, captured decode steps
    with padding rows, pipelined or not): the windowed group's pool is only as large as its
    requests can fill, so the two groups' page ids and padding pages differ; more requests
    than fit at once keep the pools turning over. Logits of every generated token against
    the plain implementation."""
    import random

    from harness import TOLERANCE, record_error
    from pulsarlm_b200 import Engine, SamplingParams
    from pulsarlm_b200.models.model import Model
    from pulsarlm_b200.weights.loader import check_tensors

    rng = random.Random(seed)
    n_kv = rng.choice([1, 2])
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2,
           "hidden_size": 128, "num_attention_heads": n_kv * rng.choice([1, 2, 4]),
           "num_key_value_heads": n_kv, "head_dim": rng.choice([64, 128]), "intermediate_size": 256,
           "vocab_size": 300, "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
           "max_position_embeddings": 8192}
    w = tiny.random_weights(cfg, seed, torch.bfloat16)
    spec = llama_spec(cfg)
    windows = {rng.choice([0, 1]): rng.choice([17, 40, 100])}
    for layer, window in windows.items():
        spec.layers[layer].mixer.params["window"] = window
    model = Model(spec, torch.bfloat16, DEV)
    model.load(check_tensors("test", model.tensor_needs(), w, torch.bfloat16, DEV))
    prompts = [tiny.random_tokens(cfg, rng.choice([5, 90, 300, 520]), 31 * seed + i) for i in range(7)]
    new_tokens, page, slots = 20, 16, 3
    portion = rng.choice([32, 64])
    engine = Engine(model, n_pages=3 * (-(-(540 + new_tokens) // page) + 1), page_size=page, max_requests=slots,
                    prefill_tokens_per_step=portion, stop_ids=[], lookahead=seed % 2 == 0, record_logits=True)
    full, windowed = (engine.cache.groups[engine.cache.layer_group[layer]] for layer in (1 - list(windows)[0],
                                                                                         list(windows)[0]))
    assert windowed.n_pages < full.n_pages and windowed.tensor.shape[1] == windowed.n_pages + 1
    requests = [engine.submit(p, sampling=SamplingParams(temperature=0.0), max_tokens=new_tokens, ignore_eos=True)
                for p in prompts]
    while any(not r.finished for r in requests):
        engine.step()
    engine.sync()
    engine.runner.check_status()
    assert engine.runner.graph_steps > 0
    assert windowed.pool.high_water <= windowed.n_pages and engine.scheduler.preemptions == 0
    for prompt, request in zip(prompts, requests):
        output = list(request.output)
        assert len(output) == new_tokens == len(request.logits)
        want = plain_variant(cfg, w, list(prompt) + output[:-1], spec.order, windows=windows)
        err = plain_llama.max_relative_error(torch.stack(request.logits), want[len(prompt) - 1:])
        record_error("bfloat16", "windowed group with a pool of its own size through the engine", err,
                     TOLERANCE["bfloat16"])
        assert err < TOLERANCE["bfloat16"], (err, cfg, windows)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("cfg_key", ["A", "B"])
def test_attention_with_per_head_norms_and_squashed_scores(dtype, tol, cfg_key):
    """Options of the attention part that Llama leaves off: an RMS norm over each head of
    q and of k before the rotation (own scales, own eps), and scores squashed by
    cap * tanh(s / cap). Layer 0 has the norms, layer 1 the cap and the norms, the rest
    is Llama's; prompts in a portion and single tokens, against the formulas written out."""
    from pulsarlm_b200.parts.spec import TensorNeed  # noqa: F401

    cfg = {"A": tiny.TINY_A, "B": tiny.TINY_B}[cfg_key]
    hd = plain_llama.head_dim_of(cfg)
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    w = tiny.random_weights(cfg, 12, dtype)
    gen = torch.Generator().manual_seed(4)
    spec = llama_spec(cfg)
    eps, cap = 1e-3, 1.5
    for layer in (0, 1):
        p = f"model.layers.{layer}.self_attn."
        spec.layers[layer].mixer.params["qk_norm_eps"] = eps
        spec.layers[layer].mixer.tensors.update({"q_norm": p + "q_norm.weight", "k_norm": p + "k_norm.weight"})
        w[p + "q_norm.weight"] = (1.0 + 0.3 * torch.randn(hd, generator=gen)).float()
        w[p + "k_norm.weight"] = (1.0 + 0.3 * torch.randn(hd, generator=gen)).float()
    spec.layers[1].mixer.params["softcap"] = cap
    tokens = tiny.random_tokens(cfg, 45, 6)
    got, _ = run_whole(spec, w, dtype, tokens)

    wd = {k: v.double() for k, v in w.items()}
    n = len(tokens)
    pos = torch.arange(n)
    rope = plain_llama.rope_settings(cfg)
    inv = plain_llama.rope_inverse_frequency(rope["theta"], hd, rope["llama3"])
    rms = cfg["rms_norm_eps"]
    x = plain_llama.embed(wd["model.embed_tokens.weight"], torch.tensor(tokens))
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        h = plain_llama.rms_norm(x, wd[p + "input_layernorm.weight"], rms)
        if layer in (0, 1):
            q = (h @ wd[p + "self_attn.q_proj.weight"].T).view(n, nh, hd)
            k = (h @ wd[p + "self_attn.k_proj.weight"].T).view(n, nkv, hd)
            v = (h @ wd[p + "self_attn.v_proj.weight"].T).view(n, nkv, hd)
            q = plain_llama.rms_norm(q, wd[p + "self_attn.q_norm.weight"], eps)
            k = plain_llama.rms_norm(k, wd[p + "self_attn.k_norm.weight"], eps)
            q, k = plain_llama.rope_rotate(q, pos, inv), plain_llama.rope_rotate(k, pos, inv)
            group = nh // nkv
            scores = torch.einsum("qhd,khd->hqk", q, k.repeat_interleave(group, dim=1)) / math.sqrt(hd)
            if layer == 1:
                scores = cap * torch.tanh(scores / cap)
            scores = scores.masked_fill(pos[None, :] > pos[:, None], float("-inf"))
            o = torch.einsum("hqk,khd->qhd", torch.softmax(scores, dim=-1), v.repeat_interleave(group, dim=1))
            x = x + o.reshape(n, nh * hd) @ wd[p + "self_attn.o_proj.weight"].T
        else:
            x = x + plain_llama.attention_block(h, wd, p, cfg, pos)
        h = plain_llama.rms_norm(x, wd[p + "post_attention_layernorm.weight"], rms)
        x = x + plain_llama.swiglu_mlp(h, wd[p + "mlp.gate_proj.weight"], wd[p + "mlp.up_proj.weight"],
                                       wd[p + "mlp.down_proj.weight"])
    head = wd.get("lm_head.weight", wd["model.embed_tokens.weight"])
    want = plain_llama.rms_norm(x, wd["model.norm.weight"], rms) @ head.T
    assert rel(got, want) < tol
