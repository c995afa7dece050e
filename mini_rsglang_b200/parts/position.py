"""Rotary position encoding, split-half pairing (j, j + d/2), every dimension rotary
(reference: crates/kernels/src/ops.cu:79-90).  The part owns the table of inverse
frequencies; the mixer's kernel computes angle = position * f_j and the rotation in float32."""
from __future__ import annotations

import torch

from .base import POSITION_ENCODINGS, PositionEncoding


@POSITION_ENCODINGS.register("rope")
class RotaryPosition(PositionEncoding):
    def __init__(self, prefix: str, head_dim: int, theta: float):
        super().__init__(prefix)
        self.head_dim, self.theta = int(head_dim), float(theta)
        self.inv_freq: torch.Tensor | None = None

    @staticmethod
    def inverse_frequencies(head_dim: int, theta: float) -> torch.Tensor:
        """f_j = 1 / float32(theta^(2j/d)): the power in float64, narrowed, then the reciprocal
        in float32 (reference: crates/kernels/src/lib.rs:612-614)."""
        j = torch.arange(head_dim // 2, dtype=torch.float64)
        power = torch.pow(torch.tensor(theta, dtype=torch.float64), 2.0 * j / head_dim)
        return 1.0 / power.to(torch.float32)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.inv_freq = self.inverse_frequencies(self.head_dim, self.theta).to(runtime.device)

    def tables(self):
        return {"inv_freq": self.inv_freq}


@POSITION_ENCODINGS.register("none")
class NoPosition(PositionEncoding):
    def __init__(self, prefix: str = ""):
        super().__init__(prefix)

    def tables(self):
        return {"inv_freq": None}
