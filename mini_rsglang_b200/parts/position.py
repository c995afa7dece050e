"""Rotary position encoding, split-half pairing (j, j + d/2), every dimension rotary
(reference: crates/kernels/src/ops.cu:79-90).  The part owns the table of inverse
frequencies; angle = position * f_j, its cosine and sine and the rotation are float32.  The
cosines and sines of a step's tokens are computed once and shared by every layer that rotates
by the same frequencies (`rotations`); kernels that have the angles at hand compute them
themselves from the frequencies of `rotation()`."""
from __future__ import annotations

import torch

from .. import kernels
from .base import POSITION_ENCODINGS, PositionEncoding, Rotation


@POSITION_ENCODINGS.register("rope")
class RotaryPosition(PositionEncoding):
    def __init__(self, prefix: str, head_dim: int, theta: float):
        super().__init__(prefix)
        self.head_dim, self.theta = int(head_dim), float(theta)
        self.inv_freq: torch.Tensor | None = None
        self.shared_key = None

    @staticmethod
    def inverse_frequencies(head_dim: int, theta: float) -> torch.Tensor:
        """f_j = 1 / float32(theta^(2j/d)): the power in float64, narrowed, then the reciprocal
        in float32 (reference: crates/kernels/src/lib.rs:612-614)."""
        j = torch.arange(head_dim // 2, dtype=torch.float64)
        power = torch.pow(torch.tensor(theta, dtype=torch.float64), 2.0 * j / head_dim)
        return 1.0 / power.to(torch.float32)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        frequencies = self.inverse_frequencies(self.head_dim, self.theta)
        self.inv_freq = frequencies.to(runtime.device)
        self.shared_key = ("rotations", frequencies.numpy().tobytes())     # layers with the same frequencies share a step's table

    def rotation(self):
        return Rotation(self.inv_freq, self.head_dim, "split_half", 1.0)

    def rotations(self, ctx):
        """[tokens, head_dim / 2, 2] float32 (cos, sin) for the step's positions; kept in `ctx.shared` for the
        step's other layers (the model empties it when a step begins)."""
        shared = getattr(ctx, "shared", None)
        if shared is not None and self.shared_key in shared:
            return shared[self.shared_key]
        table = kernels.rotation_table(ctx.positions, self.inv_freq)
        if shared is not None:
            shared[self.shared_key] = table
        return table


@POSITION_ENCODINGS.register("none")
class NoPosition(PositionEncoding):
    def __init__(self, prefix: str = ""):
        super().__init__(prefix)

    def rotation(self):
        return None

    def rotations(self, ctx):
        return None
