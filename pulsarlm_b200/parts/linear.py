"""Matrix products of the engine: y = x W^T, W stored [out, in] as checkpoints do.

float32: the library's own CUDA-core kernel (true fp32, no tensor cores, no
TF32), whose result for a row does not depend on the other rows. bfloat16:
a library matrix product (cuBLAS through torch), as the reference's engine does
for every projection (`at::linear`, pulsarlm-core/src/engine/model/llama.cpp:67-69,
81, 91, 93), with fp32 accumulation.
"""

from __future__ import annotations

import torch

from ..kernels import ops


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
        if out_dtype == torch.float32:
            # bf16 operands, fp32 accumulator written out unrounded.
            return torch.mm(x, weight.t(), out_dtype=torch.float32)
        return torch.mm(x, weight.t())
    raise ops.KernelError(f"linear: unsupported dtype {x.dtype}")
