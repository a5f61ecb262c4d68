"""Matrix products of the engine: y = x W^T, W stored [out, in] as checkpoints do.

float32: the library's own CUDA-core kernel (true fp32, no tensor cores, no
TF32), whose result for a row does not depend on the other rows. bfloat16, fp32
accumulation, by one of three routes chosen by $PULSARLM_B200_GEMM:

* "mixed" (the default): up to 16 tokens (decode steps of small batches) this
  package's own tcgen05/TMEM kernel fed by TMA (csrc/gemm_skinny.cu), which overlaps
  its set-up and first weight loads with the kernel before it; above that a library
  matrix product (cuBLAS through torch), as the reference's engine does for every
  projection (`at::linear`, pulsarlm-core/src/engine/model/llama.cpp:67-69, 81, 91,
  93);
* "tcgen05": the own kernels at every size they take (rows starting on 16 bytes):
  csrc/gemm_skinny.cu up to 64 tokens, csrc/gemm_tcgen05.cu above; the library
  elsewhere;
* "library": the library everywhere.

The default is whichever measured faster on the Llama-3.1-8B shapes; see
profiles/gemm_tcgen05_vs_library.md.
"""

from __future__ import annotations

import torch

import os

from ..kernels import ops

GEMM_ROUTE = os.environ.get("PULSARLM_B200_GEMM", "mixed")
MIXED_MAX_TOKENS = 16  # the own kernel is ahead of the library up to here
if GEMM_ROUTE not in ("library", "tcgen05", "mixed"):
    raise ValueError(f"PULSARLM_B200_GEMM must be 'library', 'tcgen05' or 'mixed', got {GEMM_ROUTE!r}")


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
        own = GEMM_ROUTE == "tcgen05" or (GEMM_ROUTE == "mixed" and tokens <= MIXED_MAX_TOKENS)
        if own and x.stride(1) == 1 and weight.stride(1) == 1 and ops.gemm_bf16_supports(
                tokens, n, k, x.stride(0) if tokens > 1 else k, weight.stride(0) if n > 1 else k):
            out = torch.empty((tokens, n), dtype=out_dtype or torch.bfloat16, device=x.device)
            ops.gemm_bf16(x, weight, out)
            return out
        if out_dtype == torch.float32:
            # bf16 operands, fp32 accumulator written out unrounded.
            return torch.mm(x, weight.t(), out_dtype=torch.float32)
        return torch.mm(x, weight.t())
    raise ops.KernelError(f"linear: unsupported dtype {x.dtype}")
