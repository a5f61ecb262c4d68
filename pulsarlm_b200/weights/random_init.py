"""Random weights from a configuration and a seed.

`random_tensors` draws every tensor the model's parts need: matrices from
N(0, std), vectors (norm scales) as 1 + N(0, vector_std). Each tensor has its
own generator seeded from (seed, tensor name), so a tensor's values do not
depend on which other tensors exist. `write_random_model` writes a model
folder (config.json, model.safetensors) that loads like any other.

The reference has random weights only inside its tests
(pulsarlm-core/tests/model/test_llama.cpp:47-79).
"""

from __future__ import annotations

import hashlib
import json
import os
from typing import Iterator

import torch

from ..parts.spec import TensorNeed
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensors(
    needs: dict[str, TensorNeed],
    seed: int,
    dtype: torch.dtype = torch.float32,
    device: torch.device | str = "cpu",
    std: float = 0.02,
    vector_std: float = 0.02,
) -> Iterator[tuple[str, torch.Tensor]]:
    """(name, tensor) for every non-optional need, drawn on `device`."""
    device = torch.device(device)
    for name, need in needs.items():
        if need.optional:
            continue
        gen = torch.Generator(device=device)
        gen.manual_seed(_tensor_seed(seed, name))
        t = torch.randn(need.shape, generator=gen, device=device, dtype=torch.float32)
        if need.role == "vector":
            t = 1.0 + vector_std * t
        else:
            t = std * t
        yield name, t.to(dtype)


def write_random_model(
    model_dir: str,
    config_text: dict,
    seed: int,
    dtype: torch.dtype = torch.float32,
    std: float = 0.02,
    vector_std: float = 0.02,
) -> str:
    """Makes `model_dir` with config.json and model.safetensors for the
    architecture `config_text` names; returns the folder."""
    from ..config.registry import read_model_config
    from ..models.model import tensor_needs_of

    arch, cfg = read_model_config(config_text)
    needs = tensor_needs_of(arch.describe(cfg))
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_text, f, indent=1)
    tensors = dict(random_tensors(needs, seed, dtype, "cpu", std, vector_std))
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return model_dir
