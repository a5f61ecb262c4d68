"""The Llama dense decoder, described as data and registered by name.

Tensor names are Hugging Face's, as the reference reads them
(pulsarlm-core/src/engine/model/llama.cpp:27-48); the layout of a layer follows
llama.cpp:61-94.
"""

from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


def describe_llama(cfg: LlamaConfig) -> ModelSpec:
    hidden = cfg.hidden_size
    rope = cfg.rope
    llama3 = None
    if rope.llama3_scaling is not None:
        s = rope.llama3_scaling
        llama3 = {
            "factor": s.factor,
            "low_freq_factor": s.low_freq_factor,
            "high_freq_factor": s.high_freq_factor,
            "original_max_position_embeddings": s.original_max_position_embeddings,
        }
    position = PartSpec("rope", {
        "theta": rope.theta,
        "head_dim": cfg.head_dim,
        "rotary_dim": 2 * int(rope.partial_rotary_factor * cfg.head_dim / 2),
        "llama3": llama3,
    })

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"hidden_size": hidden, "eps": cfg.rms_norm_eps}, {"weight": name})

    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        mixer = PartSpec(
            "attention",
            {
                "hidden_size": hidden,
                "n_heads": cfg.num_attention_heads,
                "n_kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim,
                "position": position,
                "scale": None,
                "window": None,
                "cache_from": None,
            },
            {
                "q": p + "self_attn.q_proj.weight",
                "k": p + "self_attn.k_proj.weight",
                "v": p + "self_attn.v_proj.weight",
                "o": p + "self_attn.o_proj.weight",
            },
        )
        feed_forward = PartSpec(
            "gated_mlp",
            {"hidden_size": hidden, "intermediate_size": cfg.intermediate_size, "activation": "silu"},
            {
                "gate": p + "mlp.gate_proj.weight",
                "up": p + "mlp.up_proj.weight",
                "down": p + "mlp.down_proj.weight",
            },
        )
        layers.append(LayerSpec(
            block="pre_norm",
            mixer=mixer,
            feed_forward=feed_forward,
            norms={"mixer": norm(p + "input_layernorm.weight"),
                   "feed_forward": norm(p + "post_attention_layernorm.weight")},
        ))
    sizes = {"vocab_size": cfg.vocab_size, "hidden_size": hidden}
    return ModelSpec(
        hidden_size=hidden,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("table", dict(sizes), {"weight": "model.embed_tokens.weight"}),
        layers=layers,
        order=list(range(cfg.num_hidden_layers)),
        final_norm=norm("model.norm.weight"),
        head=PartSpec("linear", dict(sizes),
                      {"weight": None, "ignored": "lm_head.weight"} if cfg.tie_word_embeddings
                      else {"weight": "lm_head.weight"}),
        eos_token_ids=cfg.eos_token_ids,
        max_position_embeddings=cfg.max_position_embeddings,
    )


register_architecture("LlamaForCausalLM", LlamaConfig.from_text, describe_llama, model_types=("llama",),
                      replace=True)
