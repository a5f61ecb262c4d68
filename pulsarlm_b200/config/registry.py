"""The one registry from an architecture's name to its configuration and model.

An architecture is two functions: `read_config(text) -> config` turns the
parsed config.json into a typed configuration, and `describe(config) ->
ModelSpec` lays the model out as data (parts, their sizes, their tensor names,
the order of layers). Everything downstream (weights, cache, step, replay)
works from the ModelSpec and never asks which architecture it came from.

The reference dispatches on the architecture string in
pulsarlm-core/src/engine/model/make_model.cpp:36-71 and routes config.json by
`model_type` in pulsarlm/src/pulsarlm/engine_model.py:253-268.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Callable

from .base import ConfigError, load_config_text


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    read_config: Callable[[dict], Any]
    describe: Callable[[Any], Any]
    model_types: tuple[str, ...] = ()


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(
    name: str,
    read_config: Callable[[dict], Any],
    describe: Callable[[Any], Any],
    model_types: tuple[str, ...] = (),
    replace: bool = False,
) -> Architecture:
    """Makes `name` (config.json's `architectures[0]`) loadable; `model_types`
    are `model_type` values that select it when `architectures` is absent."""
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    arch = Architecture(name, read_config, describe, tuple(model_types))
    _ARCHITECTURES[name] = arch
    return arch


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def find_architecture(text: dict) -> Architecture:
    """The architecture config.json names, or a ConfigError that lists what is known."""
    names = text.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    for name in names:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    model_type = text.get("model_type")
    if not names and model_type is not None:
        for arch in _ARCHITECTURES.values():
            if model_type in arch.model_types:
                return arch
    asked = names[0] if names else model_type
    raise ConfigError(
        f"config.json: unknown architecture {asked!r}; registered: {', '.join(registered_architectures()) or 'none'}"
    )


def read_model_config(text: dict) -> tuple[Architecture, Any]:
    arch = find_architecture(text)
    return arch, arch.read_config(text)


def read_model_dir(model_dir: str) -> tuple[Architecture, Any, dict]:
    """(architecture, typed config, raw config.json) of a model folder."""
    text = load_config_text(model_dir)
    arch, cfg = read_model_config(text)
    return arch, cfg, text
