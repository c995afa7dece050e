"""What a model is put together from, and the registries that name the kinds of each part.

A model is data (`models/spec.py`): an embedding, for every layer a block kind and the parts
that this kind arranges (by role: two norms, a mixer and a feed-forward for the pre-norm block),
a last norm and an output head, each a `PartSpec` (kind + parameters), and a run order.  The
classes behind the kinds are registered here.  A part gets its sizes and constants as parameters, declares
the tensors it wants (`weight_specs`), what it needs of the cache (`cache_need`,
`state_need`), takes its tensors (`bind`) and computes (`forward`).  No part knows which
model it is in: a new architecture is new specs, and new parts only where it computes
something new.

Interfaces (all tensors on the device; `ctx` is an `engine.context.StepContext`):
  Norm.forward(x) -> y                             x, y [rows, width] of the engine's dtype
  Norm.add_norm(residual, delta, rows, write_back) -> y
      residual float32 [T, width] (+ delta of the engine's dtype), normalised; the sum is
      written back unless told otherwise; `rows` picks source rows
  Embedding.forward(ctx) -> stream                 float32 [T, width] from `ctx.token_ids`
  Head.forward(hidden) -> logits                   float32 [rows, vocab]; `hidden` may be a `Prenormed`
  PositionEncoding.rotation() -> Rotation | None   how the mixer's kernel rotates: frequencies, how many of the
      head's elements turn, which elements pair, a factor on cosines and sines; None: no rotation
  PositionEncoding.rotations(ctx) -> table | None  optional: (cos, sin) of the step's tokens, made once a step
  Mixer.forward(h, ctx, cache, write_cache) -> y   h, y [T, width]; `cache` is the entry of
      `CacheStorage` that this run of the layer reads (and writes when `write_cache`)
  Mixer.step_signature(facts) -> hashable | None  optional: what, beyond the shapes, decides a step's launches
      (`facts` is a `StepFacts`); steps with fixed shapes are recorded once per signature
  FeedForward.forward(h, ctx) -> y
  Block.forward(stream, pending, ctx, cache, write_cache) -> pending
      `stream` is the float32 residual stream [T, width], updated in place; `pending` is a
      branch output not yet added (the next norm adds it), or None.  A block kind names the
      roles it arranges and the registry of each (`roles`); the layer's spec gives a part for
      every role.  The part under the role `mixer`, if any, is the one that keeps a cache.

Norms that ride on products.  With few rows a norm's own kernel costs more than its arithmetic,
so parts may opt in to two hand-overs, both optional and both invisible to parts that do not:
  * a part with `adds_to_stream = True` is given `into=ResidualLink(stream, norm)`: its last
    product may add its result to the stream itself and return a `Prenormed` (the stream times
    the norm's weights, with the rows' sums of squares) instead of a tensor;
  * a part with `takes_prenormed = True` may be handed that `Prenormed` as `h` and lets its
    first product apply the rows' factors; any other part gets `h.materialise()`, a tensor.
A block with `links_norms = True` is told the norm that follows it (`next_norm`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from ..errors import InvalidRequest
from ..weights.spec import WeightSpec


@dataclass(frozen=True)
class PartSpec:
    """A part as data: the registered kind and its parameters."""

    kind: str
    params: dict = field(default_factory=dict)


@dataclass(frozen=True)
class KVNeed:
    """A mixer that keeps keys and values in pages: all of them, or a window."""

    kv_heads: int
    head_dim: int
    kind: str = "full"       # "full" | "window"
    window: int = 0


@dataclass(frozen=True)
class StateNeed:
    """A mixer that keeps a state of fixed size per request, in the request's state slot."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class Rotation:
    """How a position encoding rotates query and key heads: element j of the first `rotary_dim` elements
    pairs with j + rotary_dim / 2 ("split_half") or the elements pair two by two ("interleaved"); pair j
    turns by position * inv_freq[j]; cosines and sines are multiplied by `magnitude`.  The kernels'
    launchers refuse what the kernels do not do (`kernels.check_rotation`)."""

    inv_freq: torch.Tensor           # [rotary_dim / 2] float32, on the device
    rotary_dim: int
    pairing: str = "split_half"
    magnitude: float = 1.0


@dataclass
class StepFacts:
    """What the host knows about a step before anything of it is on the device: the rows of every real
    sequence and where each starts in its request.  A part plans its launches from these (an attention cuts
    the sequences into tiles) and may be asked beforehand which launches a step will make
    (`step_signature`): a step whose shapes are fixed is recorded once per signature and replayed.
    `plans` keeps what was planned, by the planner's own key, for the layers that share it."""

    q_start: list[int]                 # [real sequences + 1] first row of each real sequence
    start_pos: list[int]               # [real sequences] position of its first token of this step
    longest_context: int               # tokens of the longest sequence after the step, or the class it falls in
    padded_sequences: int = 0          # sequences of a step with fixed shapes (the real ones come first), else 0
    padded_tokens: int = 0             # its rows
    plans: dict = field(default_factory=dict)


@dataclass
class Runtime:
    """Where and in which precision a model runs."""

    device: torch.device
    dtype: torch.dtype           # torch.bfloat16 (serving) or torch.float32 (the 32-bit path)
    page_size: int = 16

    @property
    def is_bf16(self) -> bool:
        return self.dtype is torch.bfloat16


@dataclass
class ResidualLink:
    """Where a branch's output goes: the float32 stream and the norm that reads it next."""

    stream: torch.Tensor
    norm: "Norm"


@dataclass
class Prenormed:
    """Rows that a norm has not finished: `scaled` = the stream times the norm's weights (in the
    engine's dtype), `square_sums` [parts, >= rows] float32 the parts of each row's sum of squares.
    A product over `scaled` whose sums are multiplied by rsqrt(sum of a row's parts / width + eps)
    is the product over the normalised rows.  The stream already holds the branch's output."""

    scaled: torch.Tensor
    square_sums: torch.Tensor
    norm: "Norm"
    stream: torch.Tensor

    @property
    def shape(self):
        return self.scaled.shape

    @property
    def row_sums(self) -> tuple:
        return (self.square_sums, self.norm.width, self.norm.eps)

    def materialise(self) -> torch.Tensor:
        """The normalised rows as a tensor (the norm's own kernel over the stream)."""
        return self.norm.add_norm(self.stream, None)


def observing(ctx) -> bool:
    """Whether the step is watched layer by layer (`StepContext.observe`); a part asked without a context is not."""
    return getattr(ctx, "observe", None) is not None


def plain(h):
    """`h` as a tensor."""
    return h.materialise() if isinstance(h, Prenormed) else h


class Part:
    """Base of every part.  `prefix` is the root of its tensor names in the checkpoint."""

    def __init__(self, prefix: str = ""):
        self.prefix = prefix
        self.runtime: Runtime | None = None

    def name(self, leaf: str) -> str:
        return f"{self.prefix}.{leaf}" if self.prefix else leaf

    def weight_specs(self) -> list[WeightSpec]:
        return []

    def bind(self, tensors: dict[str, torch.Tensor], runtime: Runtime) -> None:
        """Take the tensors named by `weight_specs` (already on the device, in their held dtype)."""
        self.runtime = runtime


class Norm(Part):
    # True when the norm is y = x * rsqrt(mean(x^2) + eps) * weight with `weight` [width] float32, `width`
    # and `eps` as attributes: a product may then take over its arithmetic (see `Prenormed`).
    rides_on_products = False

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_norm(self, residual: torch.Tensor, delta: torch.Tensor | None, rows: torch.Tensor | None = None,
                 write_back: bool = True) -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    """Token ids -> the float32 residual stream."""

    def forward(self, ctx) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    """Normalised rows -> float32 logits."""

    def forward(self, hidden) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def rotation(self) -> Rotation | None:
        raise NotImplementedError

    def rotations(self, ctx):
        """The cosines and sines of the step's tokens, [T, head_dim / 2, 2] float32, if the encoding keeps them
        for all of a step's layers; None: the mixer's kernel computes them from `rotation()`."""
        return None


class Mixer(Part):
    # True when `forward` takes everything that changes from step to step out of the context's
    # device tensors (never from its host lists): steps of single decoded tokens may then be
    # recorded once and replayed.  Padding rows of such a step have state slot -1 and write slot -1.
    replayable = False
    adds_to_stream = False        # `forward` takes `into=ResidualLink` and may return a `Prenormed`
    takes_prenormed = False       # `forward` takes a `Prenormed` as `h`

    def cache_need(self) -> KVNeed | None:
        return None

    def step_signature(self, facts: "StepFacts"):
        """What, beyond the shapes of a step, decides which kernels this mixer launches for it and with which
        grids (hashable; None: nothing).  A replayable mixer plans from `facts` only what this covers."""
        return None

    def state_need(self) -> StateNeed | None:
        return None

    def forward(self, h: torch.Tensor, ctx, cache, write_cache: bool = True) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    adds_to_stream = False
    takes_prenormed = False

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    links_norms = False           # `forward` takes `next_norm`, the norm that reads the stream after this block
    # role -> registry: the parts that this arrangement puts together, built in this order; every role is
    # also an attribute of the block.  The role `mixer`, if there is one, is the part that keeps a cache.
    roles: dict[str, "Registry"] = {}
    entry_role: str | None = None    # the role of the norm that reads the stream first (a block before this one may link to it)

    def __init__(self, prefix: str, **parts: Part):
        super().__init__(prefix)
        missing, unknown = [r for r in self.roles if r not in parts], [r for r in parts if r not in self.roles]
        if missing or unknown:
            raise InvalidRequest(f"block {type(self).__name__} at {prefix!r}: missing parts {missing}, unknown parts {unknown}")
        self.parts = {role: parts[role] for role in self.roles}
        for role, part in self.parts.items():
            setattr(self, role, part)

    @property
    def entry_norm(self):
        return self.parts.get(self.entry_role) if self.entry_role else None

    def cache_part(self):
        """The part whose `cache_need` / `state_need` this layer's cache entry serves, or None."""
        return self.parts.get("mixer")

    def children(self) -> list[Part]:
        return list(self.parts.values())

    def weight_specs(self) -> list[WeightSpec]:
        return [s for child in self.children() for s in child.weight_specs()]

    def bind(self, tensors, runtime) -> None:
        super().bind(tensors, runtime)
        for child in self.children():
            child.bind(tensors, runtime)

    def forward(self, stream, pending, ctx, cache, write_cache: bool = True):
        raise NotImplementedError


class Registry:
    """Name -> class for one kind of part."""

    def __init__(self, what: str):
        self.what = what
        self.entries: dict[str, Callable] = {}

    def register(self, kind: str, cls: Callable | None = None, replace: bool = False):
        def put(c):
            if kind in self.entries and not replace and self.entries[kind] is not c:
                raise InvalidRequest(f"{self.what} kind {kind!r} is registered already")
            self.entries[kind] = c
            return c

        return put if cls is None else put(cls)

    def get(self, kind: str) -> Callable:
        if kind not in self.entries:
            raise InvalidRequest(f"unknown {self.what} kind {kind!r}; registered: {sorted(self.entries)}")
        return self.entries[kind]

    def build(self, spec: PartSpec, prefix: str, **extra):
        return self.get(spec.kind)(prefix=prefix, **spec.params, **extra)


EMBEDDINGS = Registry("embedding")
HEADS = Registry("output head")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block")
