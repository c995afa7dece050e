"""A model as data: the parts of every layer and the order in which layers run."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping

from ..errors import InvalidRequest
from ..parts.base import BLOCKS, EMBEDDINGS, HEADS, NORMS, PartSpec
from ..weights.spec import WeightSpec


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement (`block`, a registered block kind) and a part for every role that this
    kind arranges.  `prefix` is the root of the layer's tensor names; a part's own root hangs below it
    under `names[role]` (the role itself when `names` does not give one)."""

    prefix: str
    block: str
    parts: Mapping[str, PartSpec]
    names: Mapping[str, str] = field(default_factory=dict)


def pre_norm_layer(prefix: str, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec, feed_forward: PartSpec,
                   norm1_name: str = "input_layernorm", mixer_name: str = "self_attn",
                   norm2_name: str = "post_attention_layernorm", feed_forward_name: str = "mlp") -> LayerSpec:
    """A layer of the "pre_norm" arrangement with the usual tensor-name roots."""
    return LayerSpec(prefix, "pre_norm", {"norm1": norm1, "mixer": mixer, "norm2": norm2, "feed_forward": feed_forward},
                     {"norm1": norm1_name, "mixer": mixer_name, "norm2": norm2_name, "feed_forward": feed_forward_name})


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
    embedding: PartSpec
    embedding_prefix: str
    layers: list[LayerSpec]
    final_norm: PartSpec
    final_norm_prefix: str
    head: PartSpec
    head_prefix: str
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
        embedding = EMBEDDINGS.build(self.embedding, self.embedding_prefix)
        blocks = []
        for layer in self.layers:
            kind = BLOCKS.get(layer.block)
            missing = [role for role in kind.roles if role not in layer.parts]
            unknown = [role for role in layer.parts if role not in kind.roles]
            if missing or unknown:
                raise InvalidRequest(f"layer {layer.prefix!r}: block kind {layer.block!r} arranges {sorted(kind.roles)}; "
                                     f"missing {missing}, unknown {unknown}")
            parts = {role: registry.build(layer.parts[role], f"{layer.prefix}.{layer.names.get(role, role)}")
                     for role, registry in kind.roles.items()}
            blocks.append(kind(prefix=layer.prefix, **parts))
        final_norm = NORMS.build(self.final_norm, self.final_norm_prefix)
        head = HEADS.build(self.head, self.head_prefix)
        return embedding, blocks, final_norm, head

    def weight_specs(self) -> list[WeightSpec]:
        embedding, blocks, final_norm, head = self.build_parts()
        specs = embedding.weight_specs()
        for block in blocks:
            specs += block.weight_specs()
        return specs + final_norm.weight_specs() + head.weight_specs()
