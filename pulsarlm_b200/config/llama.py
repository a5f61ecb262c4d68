"""LlamaConfig: the typed configuration of the Llama dense decoder."""

from __future__ import annotations

import dataclasses

from .base import ConfigError, RopeParameters, read_eos, read_field, read_rope, require_positive


@dataclasses.dataclass(frozen=True)
class LlamaConfig:
    """Every size and constant of a Llama dense decoder, by its config.json key.

    The reference's `dense_config` (pulsarlm-core/inc/pulsarlm/engine/model/
    dense_config.hpp:10-18) takes widths from the tensors; here they are read
    too, so that weights can be checked against them and random weights made
    from a configuration alone.
    """

    architecture: str
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope: RopeParameters
    tie_word_embeddings: bool
    max_position_embeddings: int | None
    eos_token_ids: tuple[int, ...]

    @staticmethod
    def from_text(text: dict) -> "LlamaConfig":
        """Reads config.json's keys; rejects what the engine does not compute.

        pulsarlm/src/pulsarlm/engine_model.py:237-250: biases are refused,
        `head_dim` defaults to hidden_size // num_attention_heads.
        """
        if text.get("attention_bias") or text.get("mlp_bias"):
            raise ConfigError("config.json: unsupported attention or MLP bias")
        act = text.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: unsupported hidden_act {act!r} (supported: 'silu')")
        architectures = text.get("architectures") or []
        architecture = architectures[0] if architectures else str(text.get("model_type", ""))
        n_heads = read_field(text, "num_attention_heads", int)
        hidden = read_field(text, "hidden_size", int)
        require_positive("num_attention_heads", n_heads)
        require_positive("hidden_size", hidden)
        head_dim = read_field(text, "head_dim", int, 0) or hidden // n_heads
        cfg = LlamaConfig(
            architecture=architecture,
            num_hidden_layers=read_field(text, "num_hidden_layers", int),
            hidden_size=hidden,
            num_attention_heads=n_heads,
            num_key_value_heads=read_field(text, "num_key_value_heads", int, n_heads),
            head_dim=head_dim,
            intermediate_size=read_field(text, "intermediate_size", int),
            vocab_size=read_field(text, "vocab_size", int),
            rms_norm_eps=read_field(text, "rms_norm_eps", float),
            rope=read_rope(text),
            tie_word_embeddings=read_field(text, "tie_word_embeddings", bool, False),
            max_position_embeddings=read_field(text, "max_position_embeddings", int, None),
            eos_token_ids=read_eos(text),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for name in ("num_hidden_layers", "num_key_value_heads", "head_dim", "intermediate_size", "vocab_size"):
            require_positive(name, getattr(self, name))
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"config.json: num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})"
            )
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim must be even for rotate-half RoPE, got {self.head_dim}")
        if not self.rms_norm_eps >= 0.0:
            raise ConfigError(f"config.json: rms_norm_eps must be >= 0, got {self.rms_norm_eps}")
        if self.rope.partial_rotary_factor != 1.0:
            raise ConfigError("config.json: Llama rotates whole heads (partial_rotary_factor must be 1)")

    def to_text(self) -> dict:
        """A config.json that `from_text` reads back to an equal configuration."""
        text = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope.theta,
            "rope_scaling": None,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
        }
        if self.rope.llama3_scaling is not None:
            s = self.rope.llama3_scaling
            text["rope_scaling"] = {
                "rope_type": "llama3",
                "factor": s.factor,
                "low_freq_factor": s.low_freq_factor,
                "high_freq_factor": s.high_freq_factor,
                "original_max_position_embeddings": s.original_max_position_embeddings,
            }
        if self.max_position_embeddings is not None:
            text["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_ids:
            text["eos_token_id"] = list(self.eos_token_ids)
        return text
