"""Token embedding and output head (reference: crates/kernels/src/ops.cu:15-18;
crates/models/src/qwen3.rs:232-236).  The head's logits are float32; a tied head reads the
embedding table."""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.spec import WeightSpec
from .base import EMBEDDINGS, HEADS, Embedding, Head
from .linear import linear


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):
    def __init__(self, prefix: str, vocab: int, width: int):
        super().__init__(prefix)
        self.vocab, self.width = int(vocab), int(width)
        self.table = None

    def weight_specs(self):
        return [WeightSpec(self.name("weight"), (self.vocab, self.width))]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.table = tensors[self.name("weight")]

    def forward(self, ctx) -> torch.Tensor:
        stream = torch.empty((ctx.num_tokens, self.width), dtype=torch.float32, device=self.table.device)
        kernels.embed(self.table, ctx.token_ids, stream)
        return stream


@HEADS.register("linear_head")
class OutputHead(Head):
    def __init__(self, prefix: str, vocab: int, width: int, tied_to: str | None = None):
        super().__init__(prefix)
        self.vocab, self.width, self.tied_to = int(vocab), int(width), tied_to
        self.weight = None

    def weight_specs(self):
        return [] if self.tied_to else [WeightSpec(self.name("weight"), (self.vocab, self.width))]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.tied_to if self.tied_to else self.name("weight")]

    def forward(self, hidden) -> torch.Tensor:
        """`hidden`: the normalised rows, or a `Prenormed` that the product finishes."""
        return linear(hidden, self.weight, out_dtype=torch.float32)
