"""Plain, slow Llama: whole sequences, no cache, no batching, one function per part.

This is the oracle of the test-suite. It shares no code with the package: it
reads config.json keys and tensor names directly and computes every formula
with dense torch ops on the CPU (float64 by default, so that it is more exact
than either engine path it judges).

It restates the formulas of cosmonomic/pulsarlm (each function cites the file
and lines it restates) and is anchored on the reference's own output part by
part: the reference's kernel library builds here from its unmodified sources
(baseline/ref_kernels/build.py), and tests/test_plain.py compares rms_norm, the
SwiGLU activation, rope_rotate, causal_attention (whole prompts, a portion after a
cached prefix, a single decode token; sliding window; both RoPE settings),
page_attention_mass and the argmax tie rule with outputs of those kernels recorded
on a B200 (tests/golden/reference_kernels.json), and the RoPE frequency table with
the reference's host code (tests/golden/rope_reference.json). The reference's
whole-model code (C++23, gcc 15) does not build in this image, so the order of
the parts in a layer rests on llama.cpp:84-94 as read.
"""

from __future__ import annotations

import math

import torch


# --------------------------------------------------------------------------- config

def rope_settings(cfg: dict) -> dict:
    """theta and optional llama3 scaling from either config layout.

    pulsarlm/src/pulsarlm/engine_model.py:213-234: `rope_parameters` or the older
    `rope_scaling` + `rope_theta`; type key is `rope_type` or `type`; only
    `default` and `llama3` are accepted.
    """
    params = cfg.get("rope_parameters") or cfg.get("rope_scaling") or {}
    theta = float(params.get("rope_theta") or cfg["rope_theta"])
    kind = params.get("rope_type", params.get("type", "default"))
    if kind == "default":
        return {"theta": theta, "llama3": None}
    if kind != "llama3":
        raise ValueError(f"unsupported RoPE {kind}")
    return {
        "theta": theta,
        "llama3": {
            "factor": float(params["factor"]),
            "low": float(params["low_freq_factor"]),
            "high": float(params["high_freq_factor"]),
            "original": float(params["original_max_position_embeddings"]),
        },
    }


def head_dim_of(cfg: dict) -> int:
    """pulsarlm/src/pulsarlm/engine_model.py:246: head_dim, else hidden // heads."""
    return int(cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"])


# --------------------------------------------------------------------------- parts

def rope_inverse_frequency(theta: float, head_dim: int, llama3: dict | None) -> torch.Tensor:
    """Radians per position of every pair, float64 [head_dim / 2].

    pulsarlm-core/src/kernels/rope.cpp:31-53: f_j = theta^(-2j/head_dim); with
    llama3 scaling, by wavelength 2*pi/f: shorter than original/high -> f, longer
    than original/low -> f/factor, between -> (1-s) f/factor + s f with
    s = (original/wavelength - low) / (high - low).
    """
    out = []
    for pair in range(head_dim // 2):
        f = theta ** (-2.0 * pair / head_dim)
        if llama3 is not None:
            wavelength = 2.0 * math.pi / f
            original = llama3["original"]
            if wavelength < original / llama3["high"]:
                pass
            elif wavelength > original / llama3["low"]:
                f = f / llama3["factor"]
            else:
                s = (original / wavelength - llama3["low"]) / (llama3["high"] - llama3["low"])
                f = (1.0 - s) * f / llama3["factor"] + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64)


def rope_rotate(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """rotate_half RoPE of x [tokens, heads, head_dim] at integer positions [tokens].

    pulsarlm-core/src/kernels/rope.cpp:89-98 (and tests/model/test_llama.cpp:100-111):
    angle = position * f_j in float64; first' = first cos - second sin,
    second' = second cos + first sin, the halves being [0, hd/2) and [hd/2, hd).
    """
    half = x.shape[-1] // 2
    angle = positions.to(torch.float64)[:, None] * inv_freq[None, :]
    cos = angle.cos().to(x.dtype)[:, None, :]
    sin = angle.sin().to(x.dtype)[:, None, :]
    first, second = x[..., :half], x[..., half:]
    return torch.cat([first * cos - second * sin, second * cos + first * sin], dim=-1)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """pulsarlm-core/src/kernels/rmsnorm.cu:29-49: x * rsqrt(mean(x^2) + eps) * w."""
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight.to(x.dtype)


def embed(table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """pulsarlm-core/src/engine/model/llama.cpp:86: rows of the table, unscaled."""
    return table.index_select(0, tokens)


def causal_attention(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int | None = None,
    scores_out: list | None = None
) -> torch.Tensor:
    """Dense causal softmax attention; q [T, nh, hd], k and v [T, nkv, hd] -> [T, nh, hd].

    pulsarlm-core/tests/model/test_llama.cpp:128-137 and
    src/kernels/paged_common.cu:48-54, 75-87: query head h reads kv head
    h // (nh / nkv); key j is attended by query i when j <= i (and, with a
    window w, j > i - w); scores scaled by `scale` before the softmax.
    """
    tokens, n_heads, _ = q.shape
    group = n_heads // k.shape[1]
    kh = k.repeat_interleave(group, dim=1).transpose(0, 1)  # [nh, T, hd]
    vh = v.repeat_interleave(group, dim=1).transpose(0, 1)
    qh = q.transpose(0, 1)
    scores = torch.matmul(qh, kh.transpose(1, 2)) * scale
    i = torch.arange(tokens)[:, None]
    j = torch.arange(tokens)[None, :]
    keep = j <= i
    if window is not None:
        keep = keep & (j > i - window)
    scores = scores.masked_fill(~keep, float("-inf"))
    if scores_out is not None:
        scores_out.append(scores)  # [heads, queries, keys], scaled, -inf where unattended
    probabilities = torch.softmax(scores, dim=-1)
    return torch.matmul(probabilities, vh).transpose(0, 1)


def swiglu_mlp(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """pulsarlm-core/src/engine/model/llama.cpp:91: (silu(h Wg^T) * (h Wu^T)) Wd^T."""
    g = h @ gate.T
    return ((g * torch.sigmoid(g)) * (h @ up.T)) @ down.T


def attention_block(
    h: torch.Tensor, w: dict, prefix: str, cfg: dict, positions: torch.Tensor, window: int | None = None,
    scores_out: list | None = None
) -> torch.Tensor:
    """pulsarlm-core/src/engine/model/llama.cpp:61-82: bias-free q/k/v, RoPE on q and
    k, scale 1/sqrt(head_dim), o projection."""
    n_heads = cfg["num_attention_heads"]
    n_kv = cfg["num_key_value_heads"]
    hd = head_dim_of(cfg)
    tokens = h.shape[0]
    rope = rope_settings(cfg)
    inv_freq = rope_inverse_frequency(rope["theta"], hd, rope["llama3"])
    q = (h @ w[prefix + "self_attn.q_proj.weight"].T).view(tokens, n_heads, hd)
    k = (h @ w[prefix + "self_attn.k_proj.weight"].T).view(tokens, n_kv, hd)
    v = (h @ w[prefix + "self_attn.v_proj.weight"].T).view(tokens, n_kv, hd)
    q = rope_rotate(q, positions, inv_freq)
    k = rope_rotate(k, positions, inv_freq)
    o = causal_attention(q, k, v, 1.0 / math.sqrt(hd), window, scores_out)
    return o.reshape(tokens, n_heads * hd) @ w[prefix + "self_attn.o_proj.weight"].T


# --------------------------------------------------------------------------- model

def forward(cfg: dict, weights: dict, tokens, dtype: torch.dtype = torch.float64,
            scores_out: list | None = None) -> torch.Tensor:
    """Logits [tokens, vocab] of one whole sequence starting at position 0.

    pulsarlm-core/src/engine/model/llama.cpp:84-94: embed; per layer
    x += attention(norm1(x)); x += mlp(norm2(x)); final norm; lm_head, which is
    `lm_head.weight` when the weights have one and the embedding table otherwise
    (llama.cpp:31).
    """
    w = {name: t.to(dtype) for name, t in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.shape[0])
    eps = float(cfg["rms_norm_eps"])
    x = embed(w["model.embed_tokens.weight"], tokens)
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
        x = x + attention_block(h, w, p, cfg, positions, None, scores_out)
        h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + swiglu_mlp(
            h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"]
        )
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return rms_norm(x, w["model.norm.weight"], eps) @ head.T


def greedy_generate(cfg: dict, weights: dict, prompt, n_new: int, dtype=torch.float64) -> list[int]:
    """Argmax decoding by re-running the whole sequence each token; ties go to the
    lower index (pulsarlm-core/src/kernels/gumbel_race.cu:17-21)."""
    seq = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward(cfg, weights, seq, dtype)[-1]
        best = int(torch.nonzero(logits == logits.max())[0, 0])
        out.append(best)
        seq.append(best)
    return out


def page_attention_mass(scores: torch.Tensor, portions: list, page_size: int, decay: float):
    """Per-page attention mass of one layer after feeding the sequence in `portions`
    ([first, last) position ranges, in order). scores: [heads, T, T] scaled, -inf
    where unattended. Returns (mass_sum [pages, heads], weight_sum [pages]).

    pulsarlm-core/tests/model/test_llama.cpp:150-178: a step adds, for each query p
    of the portion and each page it attends, w_p * (its largest score in the page)
    per head and w_p per page, w_p = decay * (1 - decay)^(last - 1 - p);
    src/engine/eviction.cpp:122-138: before a step's sums are added, the
    accumulators are scaled by (1 - decay)^(tokens in the step)."""
    heads, total, _ = scores.shape
    pages = -(-total // page_size)
    mass = torch.zeros(pages, heads, dtype=torch.float64)
    weight = torch.zeros(pages, dtype=torch.float64)
    for first, last in portions:
        retained = (1.0 - decay) ** (last - first)
        mass *= retained
        weight *= retained
        for p in range(first, last):
            w = decay * (1.0 - decay) ** (last - 1 - p)
            for page in range(p // page_size + 1):
                keys = scores[:, p, page * page_size : min((page + 1) * page_size, p + 1)]
                mass[page] += w * keys.max(dim=1).values
                weight[page] += w
    return mass, weight


# --------------------------------------------------------------------------- sampling

def kept_tokens(logits: torch.Tensor, temperature: float, top_k: int, top_p: float) -> torch.Tensor:
    """Boolean [vocab]: tokens a drawing row may return.

    pulsarlm-core/src/engine/sampling.cpp:50-52, 68-73: probabilities
    softmax(logits / T) ranked in descending order; a token stays while its rank
    is below top_k (0 = off) and the mass ranked above it is <= top_p (outside
    (0,1) = off).
    """
    vocab = logits.shape[0]
    p = torch.softmax(logits.double() / temperature, dim=-1)
    order = torch.argsort(p, descending=True, stable=True)
    ranked = p[order]
    keep = torch.ones(vocab, dtype=torch.bool)
    if top_k > 0:
        keep &= torch.arange(vocab) < top_k
    if 0.0 < top_p < 1.0:
        keep &= (ranked.cumsum(0) - ranked) <= top_p
    out = torch.zeros(vocab, dtype=torch.bool)
    out[order[keep]] = True
    return out


def sampling_distribution(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0):
    """Probabilities [vocab] a drawing row samples from: the kept tokens'
    softmax(logits / T), renormalised (sampling.cpp:74, the race over their logs)."""
    p = torch.softmax(logits.double() / temperature, dim=-1)
    p = p * kept_tokens(logits, temperature, top_k, top_p)
    return p / p.sum()


def max_relative_error(got: torch.Tensor, expected: torch.Tensor) -> float:
    """pulsarlm-core/tests/model/test_llama.cpp:215-217: max|got - expected| / max|expected|."""
    return float((got.double() - expected.double()).abs().max() / expected.double().abs().max())
