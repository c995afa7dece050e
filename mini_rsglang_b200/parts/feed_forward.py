"""Dense gated feed-forward: down(silu(gate(x)) * up(x)) (reference:
crates/models/src/qwen3.rs:239-262; ops.cu:91-94).  Gate and up are one projection over the
row-concatenated matrices."""
from __future__ import annotations

import torch

from .. import kernels
from ..errors import InvalidRequest
from ..weights.spec import WeightSpec
from .base import FEED_FORWARDS, FeedForward, Prenormed, observing, plain
from .linear import few_rows, linear


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    adds_to_stream = True
    takes_prenormed = True

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

    BLOCK = 64     # gate rows of a 128-row weight tile of the tensor-core product; the other 64 are the up rows

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        gate, up = tensors[self.name("gate_proj.weight")], tensors[self.name("up_proj.weight")]
        # When serving in bfloat16 and the width allows it, blocks of 64 gate rows alternate with the 64
        # matching up rows: a weight tile of the product for few rows then holds both halves of its outputs,
        # and the product applies silu(gate) * up before it stores.
        self.block = self.BLOCK if runtime.is_bf16 and self.inner % self.BLOCK == 0 else 0
        if self.block:
            b = self.block
            self.gate_up = torch.stack([gate.view(-1, b, self.width), up.view(-1, b, self.width)], dim=1) \
                .reshape(2 * self.inner, self.width).contiguous()
        else:
            self.gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.down = tensors[self.name("down_proj.weight")].contiguous()

    def forward(self, h, ctx, into=None):
        act = torch.empty((h.shape[0], self.inner), dtype=self.runtime.dtype, device=self.down.device)
        if self.block and few_rows(h, self.gate_up) and not observing(ctx):
            if isinstance(h, Prenormed):
                kernels.gemm_tc(h.scaled, self.gate_up, act, gated=True, row_sums=h.row_sums)
            else:
                kernels.gemm_tc(h, self.gate_up, act, gated=True)
        else:
            h = plain(h)
            if self.block == 64 and not observing(ctx) and kernels.gemm_gated_rows_wins(h, self.gate_up):
                kernels.gemm_gated_rows(h, self.gate_up, act)      # many rows: the tcgen05 product with the activation in it
            else:
                kernels.silu_mul(linear(h, self.gate_up), act, self.block)
        if observing(ctx):
            ctx.observe(f"{ctx.label}-swiglu", act)
        return linear(act, self.down, into=into)
