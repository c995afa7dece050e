"""A model as data: the parts of every layer and the order in which layers run."""
from __future__ import annotations

from dataclasses import dataclass, field

from ..errors import InvalidRequest
from ..parts.base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, PartSpec
from ..parts.embedding import OutputHead, TokenEmbedding
from ..weights.spec import WeightSpec


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement (`block`) and the parts it arranges.  `prefix` is the root of
    the layer's tensor names; the parts' own prefixes hang below it."""

    prefix: str
    block: str
    norm1: PartSpec
    mixer: PartSpec
    norm2: PartSpec
    feed_forward: PartSpec
    norm1_name: str = "input_layernorm"
    mixer_name: str = "self_attn"
    norm2_name: str = "post_attention_layernorm"
    feed_forward_name: str = "mlp"


@dataclass(frozen=True)
class RunEntry:
    """One run of a layer.  `cache_of` names an earlier entry of the run order whose cache this
    run reads instead of keeping one of its own (it then writes nothing)."""

    layer: int
    cache_of: int | None = None


@dataclass
class ModelSpec:
    vocab_size: int
    width: int
    embedding_prefix: str
    layers: list[LayerSpec]
    final_norm: PartSpec
    final_norm_prefix: str
    head_prefix: str
    tie_head_to_embedding: bool
    run_order: list[RunEntry] = field(default_factory=list)
    ignorable_weights: tuple[str, ...] = ()

    def __post_init__(self):
        if not self.run_order:
            self.run_order = [RunEntry(i) for i in range(len(self.layers))]
        for index, entry in enumerate(self.run_order):
            if not 0 <= entry.layer < len(self.layers):
                raise InvalidRequest(f"run order names layer {entry.layer}, the model has {len(self.layers)}")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < index or self.run_order[entry.cache_of].cache_of is not None:
                    raise InvalidRequest("cache_of must name an earlier run that keeps a cache of its own")

    def build_parts(self):
        """Instantiate every part (no tensors yet): (embedding, blocks, final norm, head)."""
        embedding = TokenEmbedding(self.embedding_prefix, self.vocab_size, self.width)
        blocks = []
        for layer in self.layers:
            blocks.append(BLOCKS.get(layer.block)(
                prefix=layer.prefix,
                norm1=NORMS.build(layer.norm1, f"{layer.prefix}.{layer.norm1_name}"),
                mixer=MIXERS.build(layer.mixer, f"{layer.prefix}.{layer.mixer_name}"),
                norm2=NORMS.build(layer.norm2, f"{layer.prefix}.{layer.norm2_name}"),
                feed_forward=FEED_FORWARDS.build(layer.feed_forward, f"{layer.prefix}.{layer.feed_forward_name}")))
        final_norm = NORMS.build(self.final_norm, self.final_norm_prefix)
        tied = f"{self.embedding_prefix}.weight" if self.tie_head_to_embedding else None
        head = OutputHead(self.head_prefix, self.vocab_size, self.width, tied_to=tied)
        return embedding, blocks, final_norm, head

    def weight_specs(self) -> list[WeightSpec]:
        embedding, blocks, final_norm, head = self.build_parts()
        specs = embedding.weight_specs()
        for block in blocks:
            specs += block.weight_specs()
        return specs + final_norm.weight_specs() + head.weight_specs()
