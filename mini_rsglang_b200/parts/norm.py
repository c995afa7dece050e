"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * weight, statistics in float32
(reference: crates/kernels/src/ops.cu:66-78).  The weight multiplies plainly (no 1 + w)."""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.spec import WeightSpec
from .base import NORMS, Norm, Prenormed


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    rides_on_products = True

    def __init__(self, prefix: str, width: int, eps: float):
        super().__init__(prefix)
        self.width, self.eps = int(width), float(eps)
        self.weight: torch.Tensor | None = None

    def weight_specs(self):
        return [WeightSpec(self.name("weight"), (self.width,), "vector")]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.name("weight")]

    def forward(self, x):
        out = torch.empty_like(x)
        kernels.rmsnorm(x, self.weight, self.eps, out)
        return out

    def add_norm(self, residual, delta, rows=None, write_back=True):
        if isinstance(delta, Prenormed):          # the stream holds the sum already
            if delta.norm is self and rows is None:
                return delta                      # and the product after this norm finishes it
            delta = None
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.width), dtype=self.runtime.dtype, device=residual.device)
        kernels.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows, write_back)
        return out
