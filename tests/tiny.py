"""Tiny Llama configurations and random weights for the tests.

The two configurations differ in every size and option: layers, width, heads
and groups (MHA vs 3:1 GQA), head size (and heads * head size != width in B),
feed-forward width (172 is no multiple of 16), vocabulary (1000 is no power of
two), RoPE base and scaling (B's llama3 bands all occur within 16 pairs), the
norms' eps, tied vs untied head, page size. Weights are drawn here with torch
and written with the `safetensors` package, not with the engine's own writer,
so the engine's reader is checked against an independent file.
"""

from __future__ import annotations

import json
import os

import torch

TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 2,
    "hidden_size": 64,
    "num_attention_heads": 4,
    "num_key_value_heads": 4,
    "head_dim": 16,
    "intermediate_size": 172,
    "vocab_size": 256,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True,
    "max_position_embeddings": 256,
    "hidden_act": "silu",
}
PAGE_A = 16

TINY_B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 3,
    "hidden_size": 96,
    "num_attention_heads": 6,
    "num_key_value_heads": 2,
    "head_dim": 32,
    "intermediate_size": 256,
    "vocab_size": 1000,
    "rope_theta": 500000.0,
    "rope_scaling": {
        "rope_type": "llama3",
        "factor": 8.0,
        "low_freq_factor": 1.0,
        "high_freq_factor": 4.0,
        "original_max_position_embeddings": 64,
    },
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "max_position_embeddings": 512,
    "hidden_act": "silu",
}
PAGE_B = 32

# A third shape for the tensor-core kernels: head size 64, 4:1 groups, untied.
TINY_C = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 2,
    "hidden_size": 160,
    "num_attention_heads": 8,
    "num_key_value_heads": 2,
    "head_dim": 64,
    "intermediate_size": 336,
    "vocab_size": 515,
    "rope_theta": 10000.0,
    "rope_scaling": {
        "rope_type": "llama3",
        "factor": 4.0,
        "low_freq_factor": 1.0,
        "high_freq_factor": 4.0,
        "original_max_position_embeddings": 128,
    },
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "max_position_embeddings": 2048,
    "hidden_act": "silu",
}
PAGE_C = 16


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    h = cfg["hidden_size"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or h // nh
    inter, vocab = cfg["intermediate_size"], cfg["vocab_size"]
    shapes = {"model.embed_tokens.weight": (vocab, h), "model.norm.weight": (h,)}
    if not cfg.get("tie_word_embeddings", False):
        shapes["lm_head.weight"] = (vocab, h)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        shapes[p + "input_layernorm.weight"] = (h,)
        shapes[p + "post_attention_layernorm.weight"] = (h,)
        shapes[p + "self_attn.q_proj.weight"] = (nh * hd, h)
        shapes[p + "self_attn.k_proj.weight"] = (nkv * hd, h)
        shapes[p + "self_attn.v_proj.weight"] = (nkv * hd, h)
        shapes[p + "self_attn.o_proj.weight"] = (h, nh * hd)
        shapes[p + "mlp.gate_proj.weight"] = (inter, h)
        shapes[p + "mlp.up_proj.weight"] = (inter, h)
        shapes[p + "mlp.down_proj.weight"] = (h, inter)
    return shapes


def random_weights(cfg: dict, seed: int, dtype: torch.dtype = torch.float32, scale: float = 1.0) -> dict:
    """Matrices N(0, 1/sqrt(in)) * scale (so activations keep unit size through the
    layers and every part matters to the logits), norm scales 1 + 0.1 N(0, 1), as
    the reference's test draws them (pulsarlm-core/tests/model/test_llama.cpp:47-79);
    rounded to `dtype`."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if len(shape) == 1:
            t = 1.0 + 0.1 * torch.randn(shape, generator=gen)
        elif name == "model.embed_tokens.weight":
            t = torch.randn(shape, generator=gen)
        else:
            t = torch.randn(shape, generator=gen) * (scale / shape[1] ** 0.5)
        out[name] = t.to(dtype)
    return out


def write_model_dir(folder: str, cfg: dict, weights: dict) -> str:
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(folder, "model.safetensors"))
    return folder


def random_tokens(cfg: dict, length: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab_size"], (length,), generator=gen).tolist()
