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
from .base import Prenormed, ResidualLink


def configure_library_products() -> None:
    """Process-wide settings of the library's products (torch's cuBLAS front end): float32 accumulation without
    reduced-precision reductions, and no TF32.  The step function sets them once when it is built
    (`ModelRunner.__init__`); they stay set for the process."""
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_tf32 = False


def few_rows(x, weight: torch.Tensor) -> bool:
    """Whether the engine's own tensor-core product takes this one."""
    scaled = x.scaled if isinstance(x, Prenormed) else x
    return scaled.shape[0] <= kernels.GEMM_TC_BEST_ROWS and kernels.gemm_tc_supported(scaled, weight)


def linear(x, weight: torch.Tensor, out_dtype: torch.dtype | None = None, into: ResidualLink | None = None):
    """x [M, K], weight [N, K] -> [M, N] in `out_dtype` (default: x's dtype).

    `x` may be a `Prenormed`: the product for few rows finishes the norm in its epilogue; otherwise the
    norm's own kernel runs first.  With `into` and few rows the product adds its result to the stream and
    returns a `Prenormed` for the norm that follows; otherwise it returns the tensor and the norm adds it."""
    if isinstance(x, Prenormed):
        if few_rows(x, weight):
            out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype or x.scaled.dtype, device=weight.device)
            return _tensor_core(x.scaled, weight, out, x.row_sums, into)
        x = x.materialise()
    out_dtype = out_dtype or x.dtype
    if x.dtype is torch.float32:
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=torch.float32, device=x.device)
        kernels.gemm_f32(x, weight, out)
        return out
    if few_rows(x, weight):
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=x.device)
        return _tensor_core(x, weight, out, None, into)
    if out_dtype is torch.float32:
        return torch.mm(x, weight.t(), out_dtype=torch.float32)
    return torch.mm(x, weight.t())


def _tensor_core(x, weight, out, row_sums, into):
    if into is None or out.dtype is not torch.bfloat16 or x.shape[0] > 32:
        kernels.gemm_tc(x, weight, out, row_sums=row_sums)
        return out
    sums = kernels.gemm_tc(x, weight, out, row_sums=row_sums, residual=(into.stream, into.norm.weight))
    return Prenormed(out, sums, into.norm, into.stream)
