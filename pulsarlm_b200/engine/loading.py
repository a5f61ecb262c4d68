"""From a model folder (or a configuration and a seed) to a Model with weights."""

from __future__ import annotations

import torch

from .. import models  # noqa: F401  (registers the architectures)
from ..config.registry import read_model_config, read_model_dir
from ..models.model import Model
from ..weights.loader import check_tensors, load_checked
from ..weights.random_init import random_tensors

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "fp32": torch.float32, "bf16": torch.bfloat16}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype must be float32 or bfloat16, got {name}")
        return name
    try:
        return DTYPES[str(name)]
    except KeyError:
        raise ValueError(f"dtype must be 'float32' or 'bfloat16', got {name!r}") from None


def load_model(model_dir: str, dtype, device="cuda:0") -> Model:
    """The model config.json names, with the folder's weights, on `device`."""
    dtype = parse_dtype(dtype)
    arch, cfg, _ = read_model_dir(model_dir)
    model = Model(arch.describe(cfg), dtype, torch.device(device))
    model.load(load_checked(model_dir, model.tensor_needs(), dtype, torch.device(device)))
    return model


def random_model(config_text: dict, seed: int, dtype, device="cuda:0", std: float = 0.02,
                 vector_std: float = 0.02) -> Model:
    """The model `config_text` describes with random weights drawn on the device
    (no files): for measurements at sizes whose files would take minutes to write."""
    dtype = parse_dtype(dtype)
    device = torch.device(device)
    arch, cfg = read_model_config(config_text)
    model = Model(arch.describe(cfg), dtype, device)
    needs = model.tensor_needs()
    tensors = dict(random_tensors(needs, seed, dtype, device, std, vector_std))
    model.load(check_tensors("random weights", needs, tensors, dtype, device))
    return model
