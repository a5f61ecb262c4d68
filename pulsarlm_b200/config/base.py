"""Typed reading of config.json: errors, field readers and the RoPE parameters.

Every size and constant the model uses comes from config.json through these
readers; nothing here or in the parts holds a default for a size.
"""

from __future__ import annotations

import dataclasses
import json
import os
from typing import Any


class ConfigError(ValueError):
    """A config.json that this engine cannot run, with the reason."""


_MISSING = object()


def read_field(text: dict, key: str, kind: type, default: Any = _MISSING) -> Any:
    """Value of `key` converted to `kind`; ConfigError if absent without a default
    or of the wrong type."""
    if key not in text or text[key] is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: missing key {key!r}")
        return default
    value = text[key]
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config.json: {key!r} must be a number, got {value!r}")
        return float(value)
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            raise ConfigError(f"config.json: {key!r} must be an integer, got {value!r}")
        return int(value)
    if kind is bool:
        if not isinstance(value, bool):
            raise ConfigError(f"config.json: {key!r} must be true or false, got {value!r}")
        return value
    if not isinstance(value, kind):
        raise ConfigError(f"config.json: {key!r} must be {kind.__name__}, got {value!r}")
    return value


def require_positive(name: str, value: int) -> None:
    if value <= 0:
        raise ConfigError(f"config.json: {name!r} must be positive, got {value}")


@dataclasses.dataclass(frozen=True)
class Llama3RopeScaling:
    """Frequency-band scaling of Llama 3.1
    (pulsarlm-core/inc/pulsarlm/kernels/rope_parameters.hpp:13-20)."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: float


@dataclasses.dataclass(frozen=True)
class RopeParameters:
    """theta, the rotated fraction of the head and optional llama3 scaling
    (pulsarlm-core/inc/pulsarlm/kernels/rope_parameters.hpp:22-31)."""

    theta: float
    partial_rotary_factor: float = 1.0
    llama3_scaling: Llama3RopeScaling | None = None


def read_rope(text: dict) -> RopeParameters:
    """RoPE parameters from `rope_parameters`, or from the `rope_scaling` and
    `rope_theta` keys that preceded it; `rope_type` (or `type`) must be `default`
    or `llama3` (pulsarlm/src/pulsarlm/engine_model.py:213-234)."""
    params = text.get("rope_parameters") or text.get("rope_scaling") or {}
    if not isinstance(params, dict):
        raise ConfigError(f"config.json: rope parameters must be an object, got {params!r}")
    if params.get("rope_theta") is not None:
        theta = read_field(params, "rope_theta", float)
    else:
        theta = read_field(text, "rope_theta", float)
    if theta <= 0.0:
        raise ConfigError(f"config.json: 'rope_theta' must be positive, got {theta}")
    partial = read_field(text, "partial_rotary_factor", float, 1.0)
    kind = params.get("rope_type", params.get("type", "default"))
    if kind == "default":
        return RopeParameters(theta=theta, partial_rotary_factor=partial)
    if kind == "llama3":
        scaling = Llama3RopeScaling(
            factor=read_field(params, "factor", float),
            low_freq_factor=read_field(params, "low_freq_factor", float),
            high_freq_factor=read_field(params, "high_freq_factor", float),
            original_max_position_embeddings=read_field(params, "original_max_position_embeddings", float),
        )
        if scaling.high_freq_factor == scaling.low_freq_factor:
            raise ConfigError("config.json: llama3 rope scaling needs high_freq_factor != low_freq_factor")
        return RopeParameters(theta=theta, partial_rotary_factor=partial, llama3_scaling=scaling)
    raise ConfigError(f"config.json: unsupported RoPE {kind!r} (supported: 'default', 'llama3')")


def read_eos(text: dict) -> tuple[int, ...]:
    """`eos_token_id`, an integer or a list of them, as a tuple
    (pulsarlm/src/pulsarlm/checkpoint.py:73-77)."""
    eos = text.get("eos_token_id")
    if eos is None:
        return ()
    if isinstance(eos, int) and not isinstance(eos, bool):
        return (eos,)
    if isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
        return tuple(eos)
    raise ConfigError(f"config.json: 'eos_token_id' must be an integer or a list of integers, got {eos!r}")


def load_config_text(model_dir: str) -> dict:
    """The parsed config.json of a model folder."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json")
    with open(path, "r", encoding="utf-8") as f:
        try:
            text = json.load(f)
        except json.JSONDecodeError as error:
            raise ConfigError(f"{path}: not valid JSON ({error})") from error
    if not isinstance(text, dict):
        raise ConfigError(f"{path}: must hold a JSON object")
    return text
