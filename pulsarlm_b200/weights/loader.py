"""Loading weights by tensor name, with one error that names everything wrong.

The parts of a model say which tensors they need (`tensor_needs`); this module
compares that with what the model folder holds before anything is copied, and
raises a single WeightsError listing missing tensors, unexpected tensors and
wrong shapes. The reference looks tensors up by name one at a time and reports
the first missing one (pulsarlm-core/src/engine/model/llama.cpp:18-23) and
converts every floating tensor to the engine's dtype on the way to the device
(pulsarlm/src/pulsarlm/checkpoint.py:255-264).

dtype rule: in a bfloat16 engine a "matrix" tensor becomes bfloat16; a "vector"
tensor stored in 32-bit stays 32-bit (16-bit ones become bfloat16); integer
tensors become int32. In a float32 engine every floating tensor becomes float32
(exactly, from any 16-bit storage).
"""

from __future__ import annotations

import torch

from ..parts.spec import TensorNeed
from .safetensors_io import SafetensorsFile, model_files


class WeightsError(ValueError):
    """The model folder's tensors do not fit the configuration."""

    def __init__(self, where: str, missing, unexpected, wrong_shape):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        lines = [f"{where}: the weights do not fit the configuration"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{name} is {list(got)}, expected {list(want)}" for name, got, want in self.wrong_shape))
        super().__init__("\n".join(lines))


def stored_dtype_for(need: TensorNeed, stored: torch.dtype, engine_dtype: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    if need.role == "vector" and stored in (torch.float32, torch.float64):
        return torch.float32
    return engine_dtype


def check_names(where: str, needs: dict[str, TensorNeed], shapes: dict[str, tuple[int, ...]]) -> None:
    """Raises WeightsError unless `shapes` (what is stored) fits `needs`."""
    missing = [n for n, need in needs.items() if n not in shapes and not need.optional]
    unexpected = [n for n in shapes if n not in needs]
    wrong = [(n, shapes[n], need.shape) for n, need in needs.items()
             if n in shapes and tuple(shapes[n]) != tuple(need.shape)]
    if missing or unexpected or wrong:
        raise WeightsError(where, missing, unexpected, wrong)


def load_checked(
    model_dir: str, needs: dict[str, TensorNeed], dtype: torch.dtype, device: torch.device
) -> dict[str, torch.Tensor]:
    """All needed tensors of the folder, checked, converted and on `device`."""
    files = [SafetensorsFile(p) for p in model_files(model_dir)]
    try:
        owner: dict[str, SafetensorsFile] = {}
        for f in files:
            for name in f.names():
                owner[name] = f
        check_names(model_dir, needs, {n: f.shape(n) for n, f in owner.items()})
        out: dict[str, torch.Tensor] = {}
        for name, need in needs.items():
            if name not in owner or need.role == "ignored":
                continue
            stored = owner[name].tensor(name)
            target = stored_dtype_for(need, stored.dtype, dtype)
            out[name] = stored.to(device=device, dtype=target, copy=True)
        return out
    finally:
        for f in files:
            f.close()


def check_tensors(where: str, needs: dict[str, TensorNeed], tensors: dict[str, torch.Tensor],
                  dtype: torch.dtype, device: torch.device) -> dict[str, torch.Tensor]:
    """Same checks and conversions for tensors already in memory (random weights
    made on the device, tests)."""
    check_names(where, needs, {n: tuple(t.shape) for n, t in tensors.items()})
    return {
        name: tensors[name].to(device=device, dtype=stored_dtype_for(need, tensors[name].dtype, dtype))
        for name, need in needs.items() if name in tensors and need.role != "ignored"
    }
