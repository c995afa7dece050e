"""How a layer's parts are arranged.  "pre_norm": x + mixer(norm1(x)), then
+ feed_forward(norm2(.)) (reference: crates/models/src/qwen3.rs:176-225).

The residual stream is float32.  A branch's output is not added by a kernel of its own: it
is handed on as `pending`, and the next norm adds it while it reads the stream anyway; or,
with few rows, the branch's last product adds it and the norm rides on the products around it
(`Prenormed` in parts/base.py)."""
from __future__ import annotations

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, Prenormed, ResidualLink, observing, plain


def _branch(part, h, stream, norm, *args):
    """Runs a mixer or feed-forward on `h`, telling it where its output goes if it can use that."""
    if isinstance(h, Prenormed) and not getattr(part, "takes_prenormed", False):
        h = plain(h)
    if getattr(part, "adds_to_stream", False) and norm is not None and getattr(norm, "rides_on_products", False):
        return part.forward(h, *args, into=ResidualLink(stream, norm))
    return part.forward(h, *args)


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    links_norms = True
    roles = {"norm1": NORMS, "mixer": MIXERS, "norm2": NORMS, "feed_forward": FEED_FORWARDS}
    entry_role = "norm1"

    def forward(self, stream, pending, ctx, cache, write_cache=True, next_norm=None):
        if observing(ctx):
            return self.forward_observed(stream, pending, ctx, cache, write_cache)
        h = self.norm1.add_norm(stream, pending)
        a = _branch(self.mixer, h, stream, self.norm2, ctx, cache, write_cache)
        h = self.norm2.add_norm(stream, a)
        return _branch(self.feed_forward, h, stream, next_norm, ctx)

    def forward_observed(self, stream, pending, ctx, cache, write_cache):
        """The same with every norm a kernel of its own and the reference's observer called on its labels
        (crates/models/src/qwen3.rs:177-226): input_norm here, the mixer's and feed-forward's inside them, output."""
        h = plain(self.norm1.add_norm(stream, pending))
        ctx.observe(f"{ctx.label}-input_norm", h)
        a = self.mixer.forward(h, ctx, cache, write_cache)
        h = plain(self.norm2.add_norm(stream, a))
        f = self.feed_forward.forward(h, ctx)
        ctx.observe(f"{ctx.label}-output", stream + f.float())
        return f
