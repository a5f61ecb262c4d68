"""Norm, position encoding, embedding, output head and the gated feed-forward.

Each takes its sizes and constants from its PartSpec and its tensors by the
names the spec gives; none knows the model around it.
"""

from __future__ import annotations

import math

import torch

from ..kernels import ops
from .linear import gated_feed_forward, linear
from .registry import BuildContext, Part, register_part
from .spec import PartSpec, TensorNeed


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """h = v * rsqrt(mean(v^2) + eps) * weight over the fp32 residual stream, with
    the pending layer output added first (v = x + delta, x updated in place).
    params: hidden_size, eps. tensors: weight [hidden_size].
    Formula: pulsarlm-core/src/kernels/rmsnorm.cu:29-49."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.eps = float(self.param("eps"))
        self.weight: torch.Tensor | None = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        return {spec.tensors["weight"]: TensorNeed((int(spec.params["hidden_size"]),), role="vector")}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.spec.tensors["weight"]].contiguous()

    def forward(self, x: torch.Tensor, delta: torch.Tensor | None = None,
                rows: torch.Tensor | None = None) -> torch.Tensor:
        n = rows.numel() if rows is not None else x.shape[0]
        out = torch.empty((n, self.hidden), dtype=self.ctx.dtype, device=x.device)
        ops.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)
        return out


def rope_inverse_frequencies(theta: float, head_dim: int, rotary_dim: int, llama3: dict | None) -> list[float]:
    """Radians per position for each rotated pair, in Python floats (fp64).

    f_j = theta^(-2j / head_dim); llama3 scaling by wavelength bands as in
    pulsarlm-core/src/kernels/rope.cpp:31-53.
    """
    out = []
    for pair in range(rotary_dim // 2):
        f = theta ** (-2.0 * pair / head_dim)
        if llama3 is not None:
            wavelength = 2.0 * math.pi / f
            original = float(llama3["original_max_position_embeddings"])
            low, high, factor = float(llama3["low_freq_factor"]), float(llama3["high_freq_factor"]), float(
                llama3["factor"])
            if wavelength < original / high:
                pass
            elif wavelength > original / low:
                f = f / factor
            else:
                smooth = (original / wavelength - low) / (high - low)
                f = (1.0 - smooth) * f / factor + smooth * f
        out.append(f)
    return out


@register_part("position", "rope")
class Rope(Part):
    """Rotate-half rotary encoding. params: theta, head_dim, rotary_dim (even,
    <= head_dim; pairs are (j, j + rotary_dim / 2), dims past rotary_dim pass
    through), llama3 (None or the four scaling numbers). No tensors."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.head_dim = int(self.param("head_dim"))
        self.rotary_dim = int(self.param("rotary_dim"))
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ValueError(f"rope: rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        freqs = rope_inverse_frequencies(float(self.param("theta")), self.head_dim, self.rotary_dim,
                                         spec.params.get("llama3"))
        self.inv_freq = torch.tensor(freqs, dtype=torch.float64, device=ctx.device)

    def table(self) -> tuple[torch.Tensor | None, int]:
        return (self.inv_freq if self.rotary_dim > 0 else None), self.rotary_dim


@register_part("position", "none")
class NoPosition(Part):
    """No position encoding: q and k are used as projected."""

    def table(self) -> tuple[torch.Tensor | None, int]:
        return None, 0


@register_part("embedding", "table")
class Embedding(Part):
    """x[t] = weight[token[t]], unscaled (pulsarlm-core/src/engine/model/llama.cpp:86),
    written as fp32 into the residual stream. params: vocab_size, hidden_size."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.vocab = int(self.param("vocab_size"))
        self.hidden = int(self.param("hidden_size"))
        self.weight: torch.Tensor | None = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        return {spec.tensors["weight"]: TensorNeed((int(spec.params["vocab_size"]), int(spec.params["hidden_size"])))}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.spec.tensors["weight"]].contiguous()

    def forward(self, tokens: torch.Tensor, batch=None) -> torch.Tensor:
        """`batch`: the step (an embedding that adds learned positions or scales by a
        constant of the configuration reads batch.pos); this one uses its status word."""
        x = torch.empty((tokens.numel(), self.hidden), dtype=torch.float32, device=tokens.device)
        ops.embed(self.weight, tokens, x, batch.status if batch is not None else None)
        return x


@register_part("head", "linear")
class Head(Part):
    """logits = h W^T in fp32. params: vocab_size, hidden_size. tensors: weight
    [vocab, hidden], or None for a head tied to the embedding table, which the
    model then hands over with `tie`. The reference ties when the weights hold
    no lm_head.weight (pulsarlm-core/src/engine/model/llama.cpp:31); here
    config.json's tie_word_embeddings decides, and the weights must agree."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.vocab = int(self.param("vocab_size"))
        self.hidden = int(self.param("hidden_size"))
        self.weight: torch.Tensor | None = None

    @property
    def tied(self) -> bool:
        return self.spec.tensors.get("weight") is None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        name = spec.tensors.get("weight")
        shape = (int(spec.params["vocab_size"]), int(spec.params["hidden_size"]))
        if name is None:
            # A tied checkpoint may still store a copy of the table under the head's
            # name; it is allowed and not read.
            ignored = spec.tensors.get("ignored")
            return {ignored: TensorNeed(shape, role="ignored", optional=True)} if ignored else {}
        return {name: TensorNeed((int(spec.params["vocab_size"]), int(spec.params["hidden_size"])))}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = tensors[self.spec.tensors["weight"]].contiguous()

    def tie(self, table: torch.Tensor) -> None:
        if tuple(table.shape) != (self.vocab, self.hidden):
            raise ValueError(f"head: cannot tie to a table of shape {tuple(table.shape)}")
        self.weight = table

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return linear(h, self.weight, out_dtype=torch.float32)


@register_part("feed_forward", "gated_mlp")
class GatedMLP(Part):
    """(act(h Wg^T) * (h Wu^T)) Wd^T with act = SiLU
    (pulsarlm-core/src/engine/model/llama.cpp:91). params: hidden_size,
    intermediate_size, activation. tensors: gate, up [I, H], down [H, I].
    gate and up are stacked into one [2I, H] operand at load."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.inter = int(self.param("intermediate_size"))
        act = spec.params.get("activation", "silu")
        if act != "silu":
            raise ValueError(f"gated_mlp: unsupported activation {act!r} (supported: 'silu')")
        self.gate_up: torch.Tensor | None = None
        self.down: torch.Tensor | None = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        h, i = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        t = spec.tensors
        return {t["gate"]: TensorNeed((i, h)), t["up"]: TensorNeed((i, h)), t["down"]: TensorNeed((h, i))}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        t = self.spec.tensors
        self.gate_up = torch.cat([tensors[t["gate"]], tensors[t["up"]]], dim=0).contiguous()
        self.down = tensors[t["down"]].contiguous()

    def forward(self, h: torch.Tensor, batch) -> torch.Tensor:
        return gated_feed_forward(h, self.gate_up, self.down)
