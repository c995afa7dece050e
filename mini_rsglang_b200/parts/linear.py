"""Matrix products y = x . W^T (W stored [out, in], no bias).

On the 32-bit path the product is the engine's own float32 kernel (CUDA-core FMA, no
reduced-precision mode).  When serving in bfloat16, up to 128 rows (decoded tokens, short
portions) go through the engine's tcgen05 kernel, which streams the weights once with bulk
tensor copies; more rows go through the library (cuBLAS through torch.mm, float32
accumulation, reduced-precision reductions switched off), as the reference uses cuBLAS for
every projection (crates/kernels/src/lib.rs:298-321)."""
from __future__ import annotations

import torch

from .. import kernels

_configured = False


def _configure_library() -> None:
    global _configured
    if not _configured:
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        torch.backends.cuda.matmul.allow_tf32 = False
        _configured = True


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """x [M, K], weight [N, K] -> [M, N] in `out_dtype` (default: x's dtype)."""
    out_dtype = out_dtype or x.dtype
    if x.dtype is torch.float32:
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=torch.float32, device=x.device)
        kernels.gemm_f32(x, weight, out)
        return out
    if x.shape[0] <= kernels.GEMM_TC_BEST_ROWS and kernels.gemm_tc_supported(x, weight):
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=x.device)
        kernels.gemm_tc(x, weight, out)
        return out
    _configure_library()
    if out_dtype is torch.float32:
        return torch.mm(x, weight.t(), out_dtype=torch.float32)
    return torch.mm(x, weight.t())
