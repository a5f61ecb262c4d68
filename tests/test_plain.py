"""The plain implementation itself: anchored on the reference's host RoPE code and
checked for the properties the engine tests rely on."""

import json
import math
import os

import torch

import plain_llama
import tiny

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "rope_reference.json")

CASES = {
    "tiny_a": (tiny.TINY_A, None),
    "tiny_b": (tiny.TINY_B, None),
    "tiny_c": (tiny.TINY_C, None),
    "llama31_8b": ({"rope_theta": 500000.0, "head_dim": 128, "hidden_size": 4096, "num_attention_heads": 32,
                    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}}, None),
}


def test_rope_table_matches_reference_host_code():
    with open(GOLDEN) as f:
        golden = json.load(f)
    for name, (cfg, _) in CASES.items():
        rope = plain_llama.rope_settings(cfg)
        hd = plain_llama.head_dim_of(cfg)
        inv_freq = plain_llama.rope_inverse_frequency(rope["theta"], hd, rope["llama3"])
        want = torch.tensor(golden[name]["quadrants_per_position"], dtype=torch.float64) * (math.pi / 2)
        assert torch.allclose(inv_freq, want, rtol=1e-14, atol=0), name


def test_rope_rotation_matches_reference_host_code():
    with open(GOLDEN) as f:
        golden = json.load(f)
    for name, (cfg, _) in CASES.items():
        rope = plain_llama.rope_settings(cfg)
        hd = plain_llama.head_dim_of(cfg)
        inv_freq = plain_llama.rope_inverse_frequency(rope["theta"], hd, rope["llama3"])
        pos = torch.tensor(golden[name]["positions"]).long()
        d = torch.arange(hd, dtype=torch.float64)
        x = torch.sin(0.37 * d[None, :] + 0.11 * pos.double()[:, None]).float()
        got = plain_llama.rope_rotate(x[:, None, :], pos, inv_freq)[:, 0, :]
        want = torch.tensor(golden[name]["rotated"], dtype=torch.float64).view(len(pos), hd)
        assert (got.double() - want).abs().max() < 2e-7, name


def test_llama3_bands_all_occur_in_tiny_b():
    rope = plain_llama.rope_settings(tiny.TINY_B)
    plain = plain_llama.rope_inverse_frequency(rope["theta"], 32, None)
    scaled = plain_llama.rope_inverse_frequency(rope["theta"], 32, rope["llama3"])
    ratio = scaled / plain
    assert (ratio == 1.0).any() and torch.isclose(ratio, torch.tensor(1 / 8.0, dtype=torch.float64)).any()
    assert ((ratio < 0.999) & (ratio > 0.126)).any()


def test_forward_is_causal_and_uses_every_part():
    cfg = tiny.TINY_B
    w = tiny.random_weights(cfg, 3)
    tokens = tiny.random_tokens(cfg, 24, 1)
    full = plain_llama.forward(cfg, w, tokens)
    prefix = plain_llama.forward(cfg, w, tokens[:10])
    assert torch.allclose(full[:10], prefix, atol=1e-12)
    for name in w:
        changed = dict(w)
        changed[name] = w[name] * 1.5 if w[name].dim() == 2 else w[name] + 0.5
        other = plain_llama.forward(cfg, changed, tokens)
        assert (other - full).abs().max() > 1e-6, f"{name} does not reach the logits"


def test_tied_head_uses_embedding():
    cfg = tiny.TINY_A
    w = tiny.random_weights(cfg, 2)
    assert "lm_head.weight" not in w
    tokens = tiny.random_tokens(cfg, 9, 4)
    logits = plain_llama.forward(cfg, w, tokens)
    untied = dict(w)
    untied["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    assert torch.equal(logits, plain_llama.forward(cfg, untied, tokens))


def test_window_limits_reach():
    q = torch.randn(12, 2, 8, dtype=torch.float64)
    k = torch.randn(12, 1, 8, dtype=torch.float64)
    v = torch.randn(12, 1, 8, dtype=torch.float64)
    full = plain_llama.causal_attention(q, k, v, 0.3)
    windowed = plain_llama.causal_attention(q, k, v, 0.3, window=4)
    assert torch.allclose(full[:4], windowed[:4])
    assert not torch.allclose(full[6:], windowed[6:])
    alone = plain_llama.causal_attention(q[8:], k[8:], v[8:], 0.3)
    assert torch.allclose(windowed[11], alone[3])  # query 11 reads keys 8..11 only


def test_kept_tokens_rules():
    logits = torch.log(torch.tensor([0.5, 0.25, 0.15, 0.07, 0.03]))
    assert plain_llama.kept_tokens(logits, 1.0, 2, 1.0).tolist() == [True, True, False, False, False]
    # mass ranked above token 2 is 0.75 <= 0.8, above token 3 is 0.9 > 0.8
    assert plain_llama.kept_tokens(logits, 1.0, 0, 0.8).tolist() == [True, True, True, False, False]
    assert plain_llama.kept_tokens(logits, 1.0, 0, 0.3).tolist() == [True, False, False, False, False]
    p = plain_llama.sampling_distribution(logits, 1.0, top_k=2)
    assert torch.allclose(p, torch.tensor([2 / 3, 1 / 3, 0, 0, 0], dtype=torch.float64))


# --------------------------------------------------------------------------- the reference's own kernels
# tests/golden/reference_kernels.json holds outputs of cosmonomic/pulsarlm's CUDA kernels (built
# unmodified, run on a B200 by tests/golden/make_reference_kernel_golden.py); the inputs are
# rebuilt here from the same formulas. Bars: the reference's own for these kernels in float32
# (pulsarlm-core/tests/kernels/test_ops.cpp: 1e-5 on norm and rope, 1e-4 on attention, 1e-3 on mass).

KERNEL_GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_kernels.json")


def _kernel_golden():
    import sys

    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    import make_reference_kernel_golden as made

    with open(KERNEL_GOLDEN) as f:
        return made, json.load(f), made.reference_kernel_inputs()


def _llama3(values):
    if values is None:
        return None
    return {"factor": values[0], "low": values[1], "high": values[2], "original": values[3]}


def test_rms_norm_matches_reference_kernel():
    made, golden, inputs = _kernel_golden()
    for case, packed in zip(inputs["rmsnorm"], golden["rmsnorm"]):
        want = made.unpack(packed).view_as(case["x"]).double()
        got = plain_llama.rms_norm(case["x"].double(), case["w"].double(), case["eps"])
        assert plain_llama.max_relative_error(got, want) < 1e-5


def test_silu_times_up_matches_reference_kernel():
    made, golden, inputs = _kernel_golden()
    x = inputs["silu_mul"]["x"].double()
    half = x.shape[1] // 2
    want = made.unpack(golden["silu_mul"]).view(x.shape[0], half).double()
    # the activation as swiglu_mlp computes it, with identity projections
    eye = torch.eye(half, dtype=torch.float64)
    got = plain_llama.swiglu_mlp(torch.cat([x[:, :half], x[:, half:]], dim=1),
                                 torch.cat([eye, torch.zeros(half, half, dtype=torch.float64)], dim=1),
                                 torch.cat([torch.zeros(half, half, dtype=torch.float64), eye], dim=1), eye)
    assert plain_llama.max_relative_error(got, want) < 1e-5


def test_rope_matches_reference_kernel():
    made, golden, inputs = _kernel_golden()
    x = inputs["rope"]["x"]  # [heads, positions, head_dim] as the reference's kernel takes it
    pos = torch.tensor(inputs["rope"]["positions"])
    for name, settings in made.ROPES.items():
        inv_freq = plain_llama.rope_inverse_frequency(settings["theta"], x.shape[2], _llama3(settings["llama3"]))
        got = plain_llama.rope_rotate(x.transpose(0, 1).double(), pos, inv_freq).transpose(0, 1)
        want = made.unpack(golden["rope"][name]).view_as(x).double()
        # float32 sine and cosine of angles up to 7e4 radians in the kernel: 1e-5 absolute on values <= 1.5
        assert (got - want).abs().max() < 1e-5, name


def _plain_attention_rows(made, inputs, rope_name, window, scores_out=None):
    a = made.ATTENTION
    settings = made.ROPES[rope_name]
    inv_freq = plain_llama.rope_inverse_frequency(settings["theta"], a["head_dim"], _llama3(settings["llama3"]))
    scale = a["scale_factor"] / math.sqrt(a["head_dim"])
    rows = []
    for seq in inputs["attention"]:
        pos = torch.arange(seq["length"])
        q = plain_llama.rope_rotate(seq["q"].double(), pos, inv_freq)
        k = plain_llama.rope_rotate(seq["k"].double(), pos, inv_freq)
        out = plain_llama.causal_attention(q, k, seq["v"].double(), scale, window, scores_out)
        rows.append(out[seq["length"] - seq["chunk"]:])
    return torch.cat(rows, dim=0)


def test_causal_attention_matches_reference_kernel():
    """Whole prompt, a portion after a cached prefix and a single decode token, over
    scattered pages, with both RoPE settings and a sliding window: the plain attention
    (keys rotated before they are stored) against the reference's scalar kernel (keys
    stored unrotated and rotated as they are read)."""
    made, golden, inputs = _kernel_golden()
    a = made.ATTENTION
    for record in golden["attention"]:
        got = _plain_attention_rows(made, inputs, record["rope"], record["window"])
        want = made.unpack(record["out"]).view(-1, a["n_heads"], a["head_dim"]).double()
        assert got.shape == want.shape
        assert plain_llama.max_relative_error(got, want) < 1e-4, (record["rope"], record["window"])


def test_attention_mass_matches_reference_kernel():
    made, golden, inputs = _kernel_golden()
    a = made.ATTENTION
    record = next(r for r in golden["attention"] if "mass_sum" in r)
    scores: list = []
    _plain_attention_rows(made, inputs, record["rope"], record["window"], scores)
    want_mass = made.unpack(record["mass_sum"]).view(-1, a["n_heads"]).double()
    want_weight = made.unpack(record["weight_sum"]).double()
    at = 0
    for seq, s, pages in zip(inputs["attention"], scores, record["pages_per_sequence"]):
        first = seq["length"] - seq["chunk"]
        mass, weight = plain_llama.page_attention_mass(s, [(first, seq["length"])], a["page_size"], a["decay"])
        assert (mass - want_mass[at:at + pages]).abs().max() < 1e-3 * max(1.0, float(want_mass.abs().max()))
        assert (weight - want_weight[at:at + pages]).abs().max() < 1e-5
        at += pages


def test_argmax_ties_go_to_the_lower_index_as_in_the_reference_kernel():
    made, golden, inputs = _kernel_golden()
    for row, want in zip(inputs["argmax"]["scores"], golden["argmax"]):
        assert int(torch.nonzero(row == row.max())[0, 0]) == want
