"""Matrix products of the engine: y = x W^T, W stored [out, in] as checkpoints do.

float32: the library's own CUDA-core kernel (true fp32, no tensor cores, no
TF32), whose result for a row does not depend on the other rows. bfloat16, fp32
accumulation, by one of three routes chosen by $PULSARLM_B200_GEMM:

* "mixed" (the default): the own tcgen05/TMEM kernels where they measured faster than
  the library, the library elsewhere. Up to 16 tokens (decode steps of small
  batches) csrc/gemm_skinny.cu, which overlaps its set-up and first weight loads
  with the kernel before it; up to 32 tokens too where the weights are 30 MB and more
  (alone the two are even there; inside a step at batch 24 and 32 the 8B shape is 4 %
  faster with it, the 13B shape 1 - 3 %, and the 1B shape, whose q/k/v and o
  projections are smaller, 3 - 4 % with it for gate/up and down only); up to 64 tokens
  where the weights are large
  (200 MB and more: a batch-64 step's gate/up projection and head, whose time is the
  weights' stream); products of at least four 256 x 256 tiles per pair of SMs with
  most of a 256-token tile filled (a prompt portion's gate/up projection, every
  projection of long portions) csrc/gemm_pair.cu, which runs a tile on two SMs
  (`cta_group::2`); in between a library matrix product (cuBLAS through torch), as
  the reference's engine does for every projection (`at::linear`,
  pulsarlm-core/src/engine/model/llama.cpp:67-69, 81, 91, 93);
* "tcgen05": the own kernels at every size they take (rows starting on 16 bytes):
  csrc/gemm_skinny.cu up to 64 tokens, csrc/gemm_pair.cu above; the library
  elsewhere;
* "library": the library everywhere.

The default is whichever measured faster on the projection shapes of Llama-3.2-1B,
Llama-3.1-8B and Llama-2-13B at 8 to 512 tokens
(`python -m pulsarlm_b200.kernels.microbench gemm --shapes T,N,K ...` times all three).
"""

from __future__ import annotations

import torch

import os

from ..kernels import ops

GEMM_ROUTE = os.environ.get("PULSARLM_B200_GEMM", "mixed")
MIXED_MAX_TOKENS = int(os.environ.get("PULSARLM_B200_SKINNY_MAX_TOKENS", "16"))  # the skinny kernel is ahead of the library up to here,
MIXED_MID_TOKENS = 32  # up to here where the weights are at least
MIXED_MID_BYTES = 30e6  # this large,
MIXED_MAX_TOKENS_LARGE = 64  # and up to here where the weights are at least
MIXED_LARGE_BYTES = 200e6  # this large;
MIXED_MIN_TILES_PER_PAIR = 4  # the pair kernel from this many 256 x 256 tiles per pair of SMs
MIXED_MIN_TOKENS_PAIR = 192  # with a token tile at least this full (at 128 tokens the library is ahead)
if GEMM_ROUTE not in ("library", "tcgen05", "mixed"):
    raise ValueError(f"PULSARLM_B200_GEMM must be 'library', 'tcgen05' or 'mixed', got {GEMM_ROUTE!r}")


_PAIRS: dict[torch.device, int] = {}


def own_kernel_for(tokens: int, n: int, device: torch.device, k: int = 0) -> str | None:
    """Which of the package's own tcgen05 kernels the route gives a [tokens, n] product
    over k to ("skinny", "pair"), or None for the library."""
    if GEMM_ROUTE == "library":
        return None
    if GEMM_ROUTE == "tcgen05":
        return "skinny" if tokens <= ops.GEMM_SKINNY_MAX_TOKENS else "pair"
    if tokens <= MIXED_MAX_TOKENS:
        return "skinny"
    if tokens <= MIXED_MID_TOKENS and 2.0 * n * k >= MIXED_MID_BYTES:
        return "skinny"
    if tokens <= MIXED_MAX_TOKENS_LARGE:
        return "skinny" if 2.0 * n * k >= MIXED_LARGE_BYTES else None
    if tokens < MIXED_MIN_TOKENS_PAIR:
        return None
    if device not in _PAIRS:
        _PAIRS[device] = torch.cuda.get_device_properties(device).multi_processor_count // 2
    tiles = -(-n // 256) * -(-tokens // 256)
    return "pair" if tiles >= MIXED_MIN_TILES_PER_PAIR * _PAIRS[device] else None


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """x [T, K] @ weight[N, K]^T -> [T, N] in x's dtype, or fp32 when asked."""
    if x.dtype != weight.dtype:
        raise ops.KernelError(f"linear: activation dtype {x.dtype} differs from weight dtype {weight.dtype}")
    tokens = x.shape[0]
    n = weight.shape[0]
    if x.dtype == torch.float32:
        out = torch.empty((tokens, n), dtype=torch.float32, device=x.device)
        ops.gemm_f32(x, weight, out)
        return out
    if x.dtype == torch.bfloat16:
        k = x.shape[1]
        kernel = own_kernel_for(tokens, n, x.device, k)
        if kernel is not None and x.stride(1) == 1 and weight.stride(1) == 1 and ops.gemm_bf16_supports(
                tokens, n, k, x.stride(0) if tokens > 1 else k, weight.stride(0) if n > 1 else k):
            out = torch.empty((tokens, n), dtype=out_dtype or torch.bfloat16, device=x.device)
            ops.gemm_bf16(x, weight, out, kernel=kernel)
            return out
        if out_dtype == torch.float32:
            # bf16 operands, fp32 accumulator written out unrounded.
            return torch.mm(x, weight.t(), out_dtype=torch.float32)
        return torch.mm(x, weight.t())
    raise ops.KernelError(f"linear: unsupported dtype {x.dtype}")


def gated_linear(x: torch.Tensor, gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) for gate_up = [Wg; Wu] stacked [2I, K] -> [T, I].

    Both products are rounded to the activation dtype before the activation. Where the
    pair kernel runs the product, the activation happens in its epilogue (the [T, 2I]
    intermediate is never written); else the product is followed by the SwiGLU kernel."""
    tokens, k = x.shape
    inter = gate_up.shape[0] // 2
    act = torch.empty((tokens, inter), dtype=x.dtype, device=x.device)
    if (x.dtype == torch.bfloat16 == gate_up.dtype and own_kernel_for(tokens, 2 * inter, x.device, k) == "pair"
            and x.stride(1) == 1 and gate_up.stride(1) == 1
            and ops.gemm_bf16_supports(tokens, inter, k, x.stride(0) if tokens > 1 else k, gate_up.stride(0))):
        ops.gemm_bf16(x, gate_up, act, kernel="pair", gated=True)
        return act
    ops.swiglu(linear(x, gate_up), act)
    return act


GATED_IN = os.environ.get("PULSARLM_B200_GATED_IN", "1") != "0"  # (0: always the SwiGLU kernel, for comparison)


def gated_feed_forward(x: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """(silu(x Wg^T) * (x Wu^T)) Wd^T -> [T, H]. For a handful of tokens in bfloat16 the down
    projection's skinny kernel forms the gated activation itself as it reads the gate/up
    projection's output (one launch fewer, the [T, I] activation never written); else
    `gated_linear` followed by `linear`."""
    tokens, k = x.shape
    inter = gate_up.shape[0] // 2
    if (GATED_IN and x.dtype == torch.bfloat16 == gate_up.dtype == down.dtype
            and tokens <= ops.GEMM_GATED_IN_MAX_TOKENS and down.stride(1) == 1
            and own_kernel_for(tokens, down.shape[0], x.device, inter) == "skinny"
            and own_kernel_for(tokens, 2 * inter, x.device, k) != "pair"
            and ops.gemm_bf16_supports(tokens, down.shape[0], inter, 2 * inter, down.stride(0))):
        out = torch.empty((tokens, down.shape[0]), dtype=x.dtype, device=x.device)
        ops.gemm_bf16_gated_in(linear(x, gate_up), down, out)
        return out
    return linear(gated_linear(x, gate_up), down)
