"""Dense gated feed-forward: down(silu(gate(x)) * up(x)) (reference:
crates/models/src/qwen3.rs:239-262; ops.cu:91-94).  Gate and up are one projection over the
row-concatenated matrices."""
from __future__ import annotations

import torch

from .. import kernels
from ..errors import InvalidRequest
from ..weights.spec import WeightSpec
from .base import FEED_FORWARDS, FeedForward
from .linear import linear


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, prefix: str, width: int, inner: int, activation: str = "silu"):
        super().__init__(prefix)
        if activation != "silu":
            raise InvalidRequest(f"activation {activation!r} is not built; only silu")
        self.width, self.inner = int(width), int(inner)
        self.gate_up = self.down = None

    def weight_specs(self):
        return [WeightSpec(self.name("gate_proj.weight"), (self.inner, self.width)),
                WeightSpec(self.name("up_proj.weight"), (self.inner, self.width)),
                WeightSpec(self.name("down_proj.weight"), (self.width, self.inner))]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.gate_up = torch.cat([tensors[self.name("gate_proj.weight")], tensors[self.name("up_proj.weight")]],
                                 dim=0).contiguous()
        self.down = tensors[self.name("down_proj.weight")].contiguous()

    def forward(self, h, ctx):
        gate_up = linear(h, self.gate_up)
        act = torch.empty((h.shape[0], self.inner), dtype=h.dtype, device=h.device)
        kernels.silu_mul(gate_up, act)
        return linear(act, self.down)
