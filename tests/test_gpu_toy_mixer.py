"""A mixer with a state of its own, a feed-forward with routing, a position encoding of another
kind, an embedding with a scale, an output head with a soft cap and a block with three norms, all
defined here and registered from outside: an architecture made of them and of the engine's
attention is built, loaded from a folder and stepped in every cutting without a change to the
package.  The toy parts compute with plain torch operations on the device; they are not part of
any model of the engine."""
import json
import os
from dataclasses import dataclass
from typing import ClassVar

import pytest
import torch

import trace_tools as T
from mini_rsglang_b200 import RuntimeConfig
from mini_rsglang_b200.config.model_config import ModelConfig
from mini_rsglang_b200.engine import ModelRunner, SequenceStep
from mini_rsglang_b200.models.registry import ARCHITECTURES, register_architecture
from mini_rsglang_b200.models.spec import LayerSpec, ModelSpec, RunEntry, pre_norm_layer
from mini_rsglang_b200.parts import BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, \
    Embedding, FeedForward, Head, Mixer, PartSpec, PositionEncoding, Rotation, StateNeed
from mini_rsglang_b200.weights import write_random_model
from mini_rsglang_b200.weights.spec import WeightSpec

pytestmark = pytest.mark.gpu


# ---------------------------------------------------------------------------------------------
# the toy parts
# ---------------------------------------------------------------------------------------------
class DecayingSum(Mixer):
    """y_t = (sum_{i<=t} decay^(t-i) h_i) . W^T: a recurrence whose state (one vector per request)
    lives in the request's state slot between steps."""

    def __init__(self, prefix, width, decay):
        super().__init__(prefix)
        self.width, self.decay = int(width), float(decay)

    def weight_specs(self):
        return [WeightSpec(self.name("mix.weight"), (self.width, self.width))]

    def state_need(self):
        return StateNeed((self.width,), torch.float32)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.w = tensors[self.name("mix.weight")]

    def forward(self, h, ctx, cache, write_cache=True):
        out = torch.empty_like(h)
        for i in range(ctx.real_sequences or ctx.num_sequences):
            a, b = ctx.host_q_start[i], ctx.host_q_start[i + 1]
            slot = ctx.host_state_slots[i]
            state = torch.zeros(self.width, device=h.device) if ctx.fresh[i] else cache.state[slot].clone()
            for t in range(a, b):
                state = state * self.decay + h[t].float()
                out[t] = (state @ self.w.float().T).to(h.dtype)
            if write_cache:
                cache.state[slot] = state
        return out


class RoutedFeedForward(FeedForward):
    """Two small experts; a token goes to the one with the larger router logit."""

    def __init__(self, prefix, width, inner):
        super().__init__(prefix)
        self.width, self.inner = int(width), int(inner)

    def weight_specs(self):
        specs = [WeightSpec(self.name("router.weight"), (2, self.width))]
        for e in range(2):
            specs += [WeightSpec(self.name(f"experts.{e}.up.weight"), (self.inner, self.width)),
                      WeightSpec(self.name(f"experts.{e}.down.weight"), (self.width, self.inner))]
        return specs

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.t = {s.name: tensors[s.name] for s in self.weight_specs()}

    def forward(self, h, ctx):
        x = h.float()
        choice = (x @ self.t[self.name("router.weight")].float().T).argmax(dim=-1)
        out = torch.zeros_like(x)
        for e in range(2):
            up = self.t[self.name(f"experts.{e}.up.weight")].float()
            down = self.t[self.name(f"experts.{e}.down.weight")].float()
            y = torch.relu(x @ up.T) @ down.T
            out = torch.where((choice == e)[:, None], y, out)
        return out.to(h.dtype)


class HalfSpeedRotary(PositionEncoding):
    """Rotary frequencies of another law (linear, not geometric): a position encoding of its own
    that the engine's attention takes through the same `rotation()`."""

    def __init__(self, prefix, head_dim, slope):
        super().__init__(prefix)
        self.head_dim, self.slope = int(head_dim), float(slope)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.inv_freq = (self.slope / (1.0 + torch.arange(self.head_dim // 2, dtype=torch.float32))).to(runtime.device)

    def rotation(self):
        return Rotation(self.inv_freq, self.head_dim)


class ScaledEmbedding(Embedding):
    """Table rows times a constant: an embedding of another kind than the engine's."""

    def __init__(self, prefix, vocab, width, scale):
        super().__init__(prefix)
        self.vocab, self.width, self.scale = int(vocab), int(width), float(scale)

    def weight_specs(self):
        return [WeightSpec(self.name("weight"), (self.vocab, self.width))]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.table = tensors[self.name("weight")]

    def forward(self, ctx):
        return self.table[ctx.token_ids.long()].float() * self.scale


class CappedHead(Head):
    """Logits squeezed into (-cap, cap) by a tanh; reads the embedding's table."""

    def __init__(self, prefix, tied_to, cap):
        super().__init__(prefix)
        self.tied_to, self.cap = tied_to, float(cap)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.tied_to]

    def forward(self, hidden):
        from mini_rsglang_b200.parts.base import plain
        logits = plain(hidden).float() @ self.weight.float().T
        return self.cap * torch.tanh(logits / self.cap)


class SandwichBlock(Block):
    """x + post_norm(mixer(norm1(x))), then + feed_forward(norm2(.)): three norms where the engine's block has two."""

    roles = {"norm1": NORMS, "mixer": MIXERS, "post_norm": NORMS, "norm2": NORMS, "feed_forward": FEED_FORWARDS}
    entry_role = "norm1"

    def forward(self, stream, pending, ctx, cache, write_cache=True):
        from mini_rsglang_b200.parts.base import plain
        h = plain(self.norm1.add_norm(stream, pending))
        a = self.post_norm.forward(self.mixer.forward(h, ctx, cache, write_cache))
        h = plain(self.norm2.add_norm(stream, a))
        return self.feed_forward.forward(h, ctx)


@dataclass
class ToyConfig(ModelConfig):
    width: int = 0
    inner: int = 0
    heads: int = 0
    head_dim: int = 0
    decay: float = 0.0
    slope: float = 0.0
    eps: float = 1e-5
    embedding_scale: float = 1.0
    logit_cap: float = 30.0
    MODEL_TYPES: ClassVar[tuple[str, ...]] = ("toy_mix",)

    @classmethod
    def from_dict(cls, raw):
        return cls(**{k: raw[k] for k in ("model_type", "architectures", "vocab_size", "max_position_embeddings",
                                          "eos_token_id", "width", "inner", "heads", "head_dim", "decay", "slope", "eps",
                                          "embedding_scale", "logit_cap")})

    def validate(self):
        pass


def toy_spec(c: ToyConfig) -> ModelSpec:
    """Three layers: recurrence + routed experts in a block with three norms, attention (linear rotary) +
    gated feed-forward, recurrence + gated feed-forward; then the attention layer once more, reading the
    cache of its first run.  The embedding has a scale and the head a soft cap."""
    norm = PartSpec("rmsnorm", {"width": c.width, "eps": c.eps})
    recurrence = PartSpec("decaying_sum", {"width": c.width, "decay": c.decay})
    attention = PartSpec("gqa_attention", {"width": c.width, "num_heads": c.heads, "num_kv_heads": 1,
                                           "head_dim": c.head_dim,
                                           "position": PartSpec("linear_rotary", {"head_dim": c.head_dim, "slope": c.slope})})
    routed = PartSpec("routed_pair", {"width": c.width, "inner": c.inner})
    gated = PartSpec("swiglu", {"width": c.width, "inner": c.inner})
    layers = [LayerSpec("layers.0", "sandwich",
                        {"norm1": norm, "mixer": recurrence, "post_norm": norm, "norm2": norm, "feed_forward": routed},
                        {"norm1": "input_layernorm", "post_norm": "post_mixer_norm", "norm2": "post_attention_layernorm",
                         "feed_forward": "mlp"}),
              pre_norm_layer("layers.1", norm, attention, norm, gated),
              pre_norm_layer("layers.2", norm, recurrence, norm, gated, mixer_name="mixer")]
    return ModelSpec(vocab_size=c.vocab_size, width=c.width,
                     embedding=PartSpec("scaled_embedding", {"vocab": c.vocab_size, "width": c.width, "scale": c.embedding_scale}),
                     embedding_prefix="embed", layers=layers, final_norm=norm, final_norm_prefix="norm",
                     head=PartSpec("capped_head", {"tied_to": "embed.weight", "cap": c.logit_cap}), head_prefix="head",
                     run_order=[RunEntry(0), RunEntry(1), RunEntry(2), RunEntry(1, cache_of=1)])


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    MIXERS.register("decaying_sum", DecayingSum, replace=True)
    FEED_FORWARDS.register("routed_pair", RoutedFeedForward, replace=True)
    POSITION_ENCODINGS.register("linear_rotary", HalfSpeedRotary, replace=True)
    EMBEDDINGS.register("scaled_embedding", ScaledEmbedding, replace=True)
    HEADS.register("capped_head", CappedHead, replace=True)
    BLOCKS.register("sandwich", SandwichBlock, replace=True)
    register_architecture("toy_mix", ToyConfig, toy_spec, replace=True)
    config = ToyConfig(model_type="toy_mix", architectures=["ToyMix"], vocab_size=97, max_position_embeddings=256,
                       eos_token_id=1, width=40, inner=56, heads=2, head_dim=16, decay=0.8, slope=0.3, eps=1e-5,
                       embedding_scale=3.0, logit_cap=2.5)
    folder = str(tmp_path_factory.mktemp("toy"))
    write_random_model(folder, config, seed=5, dtype=torch.float32)
    yield folder
    ARCHITECTURES.pop("toy_mix", None)
    for registry, kind in ((MIXERS, "decaying_sum"), (FEED_FORWARDS, "routed_pair"), (POSITION_ENCODINGS, "linear_rotary"),
                           (EMBEDDINGS, "scaled_embedding"), (HEADS, "capped_head"), (BLOCKS, "sandwich")):
        registry.entries.pop(kind, None)


# ---------------------------------------------------------------------------------------------
# the same model, whole sequences, plain torch in float64
# ---------------------------------------------------------------------------------------------
def plain_toy(folder, tokens):
    from safetensors.torch import load_file
    w = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    with open(os.path.join(folder, "config.json")) as f:
        c = json.load(f)
    n, width, d, heads = len(tokens), c["width"], c["head_dim"], c["heads"]

    def norm(x, name):
        return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + c["eps"]) * w[name]

    def recurrence(h, root):
        state, out = torch.zeros(width, dtype=torch.float64), []
        for t in range(n):
            state = state * c["decay"] + h[t]
            out.append(state @ w[f"{root}.mixer.mix.weight"].T)
        return torch.stack(out)

    kept = {}      # keys and values of the attention layer's first run; its second run reads them

    def attention(h, root):
        q = (h @ w[f"{root}.self_attn.q_proj.weight"].T).view(n, heads, d)
        k = (h @ w[f"{root}.self_attn.k_proj.weight"].T).view(n, 1, d)
        v = (h @ w[f"{root}.self_attn.v_proj.weight"].T).view(n, 1, d)
        freq = (c["slope"] / (1.0 + torch.arange(d // 2, dtype=torch.float32))).double()
        angle = torch.arange(n, dtype=torch.float64)[:, None] * freq[None, :]
        cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]

        def rotate(x):
            a, z = x[..., :d // 2], x[..., d // 2:]
            return torch.cat([a * cos - z * sin, z * cos + a * sin], dim=-1)

        q, k = rotate(q), rotate(k)
        if root in kept:
            k, v = kept[root]
        else:
            kept[root] = (k, v)
        out = torch.empty(n, heads, d, dtype=torch.float64)
        mask = torch.tril(torch.ones(n, n, dtype=torch.bool))
        for head in range(heads):
            s = (q[:, head] @ k[:, 0].T) / d ** 0.5
            out[:, head] = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ v[:, 0]
        return out.reshape(n, heads * d) @ w[f"{root}.self_attn.o_proj.weight"].T

    def routed(h, root):
        choice = (h @ w[f"{root}.mlp.router.weight"].T).argmax(-1)
        out = torch.zeros_like(h)
        for e in range(2):
            y = torch.relu(h @ w[f"{root}.mlp.experts.{e}.up.weight"].T) @ w[f"{root}.mlp.experts.{e}.down.weight"].T
            out = torch.where((choice == e)[:, None], y, out)
        return out

    def gated(h, root):
        g, u = h @ w[f"{root}.mlp.gate_proj.weight"].T, h @ w[f"{root}.mlp.up_proj.weight"].T
        return (g / (1 + torch.exp(-g)) * u) @ w[f"{root}.mlp.down_proj.weight"].T

    x = w["embed.weight"][torch.tensor(tokens)] * c["embedding_scale"]
    for layer, mixer, ff in ((0, recurrence, routed), (1, attention, gated), (2, recurrence, gated), (1, attention, gated)):
        root = f"layers.{layer}"
        branch = mixer(norm(x, f"{root}.input_layernorm.weight"), root)
        if layer == 0:                 # the block with three norms
            branch = norm(branch, f"{root}.post_mixer_norm.weight")
        x = x + branch
        x = x + ff(norm(x, f"{root}.post_attention_layernorm.weight"), root)
    logits = norm(x, "norm.weight") @ w["embed.weight"].T
    return c["logit_cap"] * torch.tanh(logits / c["logit_cap"])


def test_toy_architecture_is_registered_built_and_stepped(toy_folder):
    limits = RuntimeConfig(max_seq_len=256, page_size=4, max_running=3)
    runner = ModelRunner.load(toy_folder, dtype="float32", limits=limits, num_pages=40)
    # the recurrences have state arrays and no pages; the attention has pages; its second run borrows them
    entries = runner.storage.entries
    assert [e.state is not None for e in entries] == [True, False, True, False]
    assert [e.k is not None for e in entries] == [False, True, False, False]
    assert entries[0].state.shape == (3, 40) and not runner.record_decode
    vocab = 97
    reqs = T.requests_for(vocab, [30, 21, 9], seed=3)
    want = {r: plain_toy(toy_folder, t) for r, t in reqs.items()}
    ids = {r: i + 1 for i, r in enumerate(reqs)}

    # each request whole
    for r, tokens in reqs.items():
        runner.cache.open(ids[r])
        runner.cache.extend(ids[r], len(tokens))
        got = runner.step([SequenceStep(ids[r], tokens, 0, list(range(len(tokens))))]).double().cpu()
        T.check_rows(got, want[r], "float32", f"toy {r} whole")
        runner.cache.close(ids[r])

    # all three together in portions of changing size, the shortest one decoding beside the others
    fed = {r: 0 for r in reqs}
    for r in reqs:
        runner.cache.open(ids[r])
    sizes = {"r0": [7, 2, 5, 1, 1, 3, 11], "r1": [2, 3, 1, 9, 1, 5], "r2": [1, 1, 1, 1, 1, 1, 1, 1, 1]}
    step = 0
    while any(fed[r] < len(reqs[r]) for r in reqs):
        batch, rows = [], []
        for r in reqs:
            if fed[r] >= len(reqs[r]):
                continue
            n = min(sizes[r][step % len(sizes[r])], len(reqs[r]) - fed[r])
            runner.cache.extend(ids[r], fed[r] + n)
            batch.append(SequenceStep(ids[r], reqs[r][fed[r]:fed[r] + n], fed[r], [n - 1]))
            rows.append((r, fed[r] + n - 1))
            fed[r] += n
        got = runner.step(batch).double().cpu()
        T.check_rows(got, torch.stack([want[r][p] for r, p in rows]), "float32", f"toy mixed step {step}")
        step += 1
    for r in reqs:
        runner.cache.close(ids[r])
    runner.cache.check_integrity()


# ---------------------------------------------------------------------------------------------
# layers with different needs of the cache: a window of keys beside all keys
# ---------------------------------------------------------------------------------------------
@dataclass
class WindowConfig(ModelConfig):
    width: int = 0
    inner: int = 0
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    theta: float = 10000.0
    eps: float = 1e-6
    MODEL_TYPES: ClassVar[tuple[str, ...]] = ("toy_window",)

    @classmethod
    def from_dict(cls, raw):
        return cls(**{k: raw[k] for k in ("model_type", "architectures", "vocab_size", "max_position_embeddings",
                                          "eos_token_id", "width", "inner", "heads", "kv_heads", "head_dim", "window",
                                          "theta", "eps")})

    def validate(self):
        pass


def window_spec(c: WindowConfig) -> ModelSpec:
    """Two attention layers: the first sees the last `window` keys only, the second all of them."""
    norm = PartSpec("rmsnorm", {"width": c.width, "eps": c.eps})
    head_norm = PartSpec("rmsnorm", {"width": c.head_dim, "eps": c.eps})

    def attention(window):
        return PartSpec("gqa_attention", {"width": c.width, "num_heads": c.heads, "num_kv_heads": c.kv_heads,
                                          "head_dim": c.head_dim, "q_norm": head_norm, "k_norm": head_norm, "window": window,
                                          "position": PartSpec("rope", {"head_dim": c.head_dim, "theta": c.theta})})

    gated = PartSpec("swiglu", {"width": c.width, "inner": c.inner})
    layers = [pre_norm_layer("model.layers.0", norm, attention(c.window), norm, gated),
              pre_norm_layer("model.layers.1", norm, attention(0), norm, gated)]
    table = {"vocab": c.vocab_size, "width": c.width}
    return ModelSpec(vocab_size=c.vocab_size, width=c.width, embedding=PartSpec("token_embedding", table),
                     embedding_prefix="model.embed_tokens", layers=layers, final_norm=norm, final_norm_prefix="model.norm",
                     head=PartSpec("linear_head", dict(table, tied_to=None)), head_prefix="lm_head")


def plain_window(folder, tokens, window_of_layer):
    import plain_qwen3 as P
    from safetensors.torch import load_file
    w = load_file(os.path.join(folder, "model.safetensors"))
    with open(os.path.join(folder, "config.json")) as f:
        c = json.load(f)
    ar = P.Arith(None)
    n, nq, nkv, d = len(tokens), c["heads"], c["kv_heads"], c["head_dim"]
    positions = torch.arange(n)
    x = P.embedding(ar, w["model.embed_tokens.weight"], torch.tensor(tokens)).double()
    for layer, window in enumerate(window_of_layer):
        root = f"model.layers.{layer}"
        h = P.rms_norm(ar, x, w[f"{root}.input_layernorm.weight"], c["eps"])
        q = P.linear(ar, h, w[f"{root}.self_attn.q_proj.weight"]).view(n, nq, d)
        k = P.linear(ar, h, w[f"{root}.self_attn.k_proj.weight"]).view(n, nkv, d)
        v = P.linear(ar, h, w[f"{root}.self_attn.v_proj.weight"]).view(n, nkv, d)
        q = P.rope(ar, P.rms_norm(ar, q, w[f"{root}.self_attn.q_norm.weight"], c["eps"]), positions, c["theta"])
        k = P.rope(ar, P.rms_norm(ar, k, w[f"{root}.self_attn.k_norm.weight"], c["eps"]), positions, c["theta"])
        a = P.causal_attention(ar, q, k, v, window).reshape(n, nq * d)
        x = x + P.linear(ar, a, w[f"{root}.self_attn.o_proj.weight"])
        h = P.rms_norm(ar, x, w[f"{root}.post_attention_layernorm.weight"], c["eps"])
        x = x + P.feed_forward_part(ar, w, root, h)
    x = P.rms_norm(ar, x, w["model.norm.weight"], c["eps"])
    return P.linear(ar, x, w["lm_head.weight"], round_out=False)


@pytest.mark.parametrize("one_wanted", [False, True])
@pytest.mark.parametrize("dtype,head_dim", [("float32", 32), ("bfloat16", 64), ("bfloat16", 32)])
def test_window_layers_have_pages_of_their_own_and_give_them_back(tmp_path, dtype, head_dim, one_wanted):
    """A layer that sees a window of keys beside one that sees all: two page groups, the window group's
    pages go back to its pool while the request runs (its block table gets holes), the pool is far
    smaller than the request and is used again and again, and the logits equal the plain ones.  Head
    size 64 runs the kernels fed by bulk tensor copies and the tcgen05 kernel with a window.  With one wanted place
    a step the steps are recorded with fixed shapes: the two layers plan tile lists of their own (a window's first
    key differs), both travel with the step's layout, and recordings are replayed over block tables with holes."""
    register_architecture("toy_window", WindowConfig, window_spec, replace=True)
    try:
        window, page = 24, 8
        config = WindowConfig(model_type="toy_window", architectures=["ToyWindow"], vocab_size=211, max_position_embeddings=1024,
                              eos_token_id=1, width=64, inner=128, heads=4, kv_heads=2, head_dim=head_dim, window=window)
        folder = str(tmp_path / "window")
        write_random_model(folder, config, seed=8, dtype=torch.bfloat16)
        limits = RuntimeConfig(max_seq_len=512, page_size=page, max_running=2, prefill_budget=64)
        runner = ModelRunner.load(folder, dtype=dtype, limits=limits, num_pages=64)
        assert [g.kind for g in runner.groups] == ["window", "full"] and runner.groups[0].window == window
        tokens = T.requests_for(211, [300], seed=2)["r0"]
        want = plain_window(folder, tokens, [window, 0])
        cache = runner.cache
        cache.open(1)
        fed, step, least_free = 0, 0, cache.free_pages(0)
        sizes = [40, 3, 1, 1, 17, 64, 1, 2, 33, 1, 1, 1, 50, 9]
        while fed < len(tokens):
            n = min(sizes[step % len(sizes)], len(tokens) - fed)
            cache.extend(1, fed + n)
            least_free = min(least_free, cache.free_pages(0))
            places = [n - 1] if one_wanted else [0, n - 1]
            got = runner.step([SequenceStep(1, tokens[fed:fed + n], fed, places)]).double().cpu()
            T.check_rows(got, want[[fed + p for p in places]], dtype, f"window model, {dtype}, head {head_dim}, step {step}")
            fed += n
            cache.trim(1, fed)
            cache.check_integrity()
            step += 1
        table = cache.table(1, 0)
        assert (table[: (fed - window) // page] < 0).all() and (table[-(window // page):] >= 0).all()
        assert (cache.table(1, 1) >= 0).all()
        held = cache.total_pages(0) - cache.free_pages(0)
        assert held <= -(-(window - 1) // page) + 1                      # only the window's pages are held at the end
        assert cache.total_pages(0) - least_free <= -(-(window - 1 + 64) // page) + 1 < len(tokens) // page
        cache.close(1)
        cache.check_integrity()
        fixed = [key for key in runner._records if len(key) == 5]
        if one_wanted:
            assert fixed and runner.recorded_steps == step
            if dtype == "bfloat16":          # a plan a layer: the window's tile lists are not the full layer's
                assert all(len(runner._records[key].ctx.plan_views) == 2 for key in fixed)
        else:
            assert not fixed
    finally:
        ARCHITECTURES.pop("toy_window", None)
