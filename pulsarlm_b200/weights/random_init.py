"""Random weights from a configuration and a seed.

`random_tensors` draws every tensor the model's parts need: matrices as std *
noise, vectors (norm scales) as 1 + vector_std * noise, the noise close to N(0, 1).
A value is a function of (seed, hash of the tensor's name, element index) alone (a
counter-based generator, csrc/random_values.h), computed by the host core for CPU
tensors and by a kernel for device tensors with identical bits: a tensor does not
depend on which other tensors exist, and a model drawn on the device for a
measurement is the model that `write_random_model` writes for the same
configuration and seed. `write_random_model` writes a model folder (config.json,
model.safetensors) that loads like any other.

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


def tensor_hash(name: str) -> int:
    """64 bits of the tensor's name: its stream among the seed's."""
    return int.from_bytes(hashlib.sha256(name.encode("utf-8")).digest()[:8], "little")


def fill_random(out: torch.Tensor, seed: int, name: str, scale: float, offset: float = 0.0) -> torch.Tensor:
    """out (float32 or bfloat16, contiguous) = offset + scale * noise(seed, name, index), in
    place; on the CPU by the host core, on a CUDA device by the kernel library."""
    if out.dtype not in (torch.float32, torch.bfloat16) or not out.is_contiguous():
        raise ValueError("fill_random takes contiguous float32 or bfloat16 tensors")
    code = 0 if out.dtype == torch.float32 else 1
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    if out.is_cuda:
        from ..kernels import ops

        ops.fill_random(out, seed, tensor_hash(name), scale, offset)
    else:
        from ..host import core

        if core.library().plh_fill_random(out.data_ptr(), out.numel(), code, seed, tensor_hash(name), scale, offset):
            raise ValueError("fill_random: the host core refused the arguments")
    return out


def random_tensors(
    needs: dict[str, TensorNeed],
    seed: int,
    dtype: torch.dtype = torch.float32,
    device: torch.device | str = "cpu",
    std: float = 0.02,
    vector_std: float = 0.02,
) -> Iterator[tuple[str, torch.Tensor]]:
    """(name, tensor) for every non-optional need, drawn on `device`. Values are made in
    float32 and rounded once to `dtype`."""
    device = torch.device(device)
    for name, need in needs.items():
        if need.optional:
            continue
        t = torch.empty(need.shape, dtype=dtype, device=device)
        if need.role == "vector":
            fill_random(t, seed, name, vector_std, 1.0)
        else:
            fill_random(t, seed, name, std)
        yield name, t


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
