"""How a layer's parts are arranged.  "pre_norm": x + mixer(norm1(x)), then
+ feed_forward(norm2(.)) (reference: crates/models/src/qwen3.rs:176-225).

The residual stream is float32.  A branch's output is not added by a kernel of its own: it
is handed on as `pending`, and the next norm adds it while it reads the stream anyway."""
from __future__ import annotations

from .base import BLOCKS, Block


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    def forward(self, stream, pending, ctx, cache, write_cache=True):
        h = self.norm1.add_norm(stream, pending)
        a = self.mixer.forward(h, ctx, cache, write_cache)
        h = self.norm2.add_norm(stream, a)
        return self.feed_forward.forward(h, ctx)
