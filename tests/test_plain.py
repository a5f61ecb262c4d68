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
