"""Each part of a layer alone, built through its registry with sizes of its own (none of them a
tiny configuration's), against the plain implementation's function for the same part."""
import pytest
import torch

import plain_qwen3 as P
from mini_rsglang_b200.cache.storage import CacheEntry
from mini_rsglang_b200.engine.context import StepContext
from mini_rsglang_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, PartSpec, Runtime
from mini_rsglang_b200.parts.embedding import OutputHead, TokenEmbedding

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
DEV = "cuda:0"


def runtime(dtype, page=8):
    return Runtime(torch.device(DEV), dtype, page)


def draw(shape, seed, std=0.05, mean=0.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g) * std + mean


def close(got, want, dtype, what):
    """float32: rounding of a float32 sum; bfloat16: one rounding of the output and of the inputs."""
    got, want = got.double().cpu(), want.double()
    scale = max(want.abs().max().item(), 1e-6)
    err = (got - want).abs().max().item()
    limit = 2e-5 * scale if dtype is torch.float32 else 2e-2 * scale
    assert err <= limit, f"{what}: max error {err:.3e} over scale {scale:.3e} ({dtype})"


def whole_sequence_context(tokens: int, page: int, first_position: int = 0, table=None):
    """The context of one request that brings `tokens` tokens from `first_position` on, its pages
    in scrambled order."""
    pages_needed = -(-(first_position + tokens) // page)
    if table is None:
        table = torch.randperm(pages_needed + 3, generator=torch.Generator().manual_seed(3))[:pages_needed]
    pos = torch.arange(first_position, first_position + tokens)
    slots = table[pos // page] * page + pos % page
    i32 = lambda x: torch.as_tensor(x, dtype=torch.int32).to(DEV)   # noqa: E731
    ctx = StepContext(
        num_tokens=tokens, num_sequences=1, token_ids=i32([0] * tokens), positions=i32(pos),
        seq_of_token=i32([0] * tokens), q_start=i32([0, tokens]), context_len=i32([first_position + tokens]),
        state_slots=i32([0]), want_rows=None, block_tables=[i32(table).view(1, -1)], slots=[i32(slots)],
        host_q_start=[0, tokens], host_start_pos=[first_position], host_state_slots=[0], max_query_len=tokens,
        max_context_len=first_position + tokens, fresh=[first_position == 0])
    return ctx, table


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    width, eps = 200, 3e-5
    norm = NORMS.build(PartSpec("rmsnorm", {"width": width, "eps": eps}), "n")
    assert [(s.name, s.shape, s.role) for s in norm.weight_specs()] == [("n.weight", (width,), "vector")]
    w = draw((width,), 1, 0.1, 1.0)
    norm.bind({"n.weight": w.to(DEV)}, runtime(dtype))
    x = draw((7, width), 2, 1.0).to(dtype)
    want = P.rms_norm(P.Arith(None), x.double(), w, eps)
    close(norm.forward(x.to(DEV)), want, dtype, "norm.forward")
    # add_norm: the float32 stream takes the branch's output while it is normalised
    stream = draw((7, width), 3, 1.0).to(DEV)
    before = stream.clone()
    delta = draw((7, width), 4, 0.5).to(dtype)
    got = norm.add_norm(stream, delta.to(DEV))
    summed = before.double().cpu() + delta.double()
    close(stream, summed, torch.float32, "stream after add_norm")
    close(got, P.rms_norm(P.Arith(None), summed, w, eps), dtype, "add_norm")
    rows = torch.tensor([5, 0], dtype=torch.int32, device=DEV)
    kept = stream.clone()
    picked = norm.add_norm(stream, delta.to(DEV), rows=rows, write_back=False)
    assert torch.equal(stream, kept), "write_back=False must leave the stream alone"
    close(picked, P.rms_norm(P.Arith(None), (kept.double().cpu() + delta.double())[[5, 0]], w, eps), dtype, "rows")


def test_rotary_part_states_its_rotation():
    for d, theta in ((48, 50000.0), (128, 1e6)):
        rope = POSITION_ENCODINGS.build(PartSpec("rope", {"head_dim": d, "theta": theta}), "p")
        assert rope.weight_specs() == []
        rope.bind({}, runtime(torch.float32))
        rotation = rope.rotation()
        assert torch.equal(rotation.inv_freq.double().cpu(), P.rope_inverse_frequencies(d, theta))
        assert (rotation.rotary_dim, rotation.pairing, rotation.magnitude) == (d, "split_half", 1.0)
    none = POSITION_ENCODINGS.build(PartSpec("none", {}), "p")
    assert none.rotation() is None and none.rotations(None) is None


def test_a_rotation_that_the_kernels_do_not_compute_is_refused_when_the_mixer_takes_its_tensors():
    """Another pairing, a rotation of part of a head and scaled cosines are a position encoding's to state and the
    kernels' launchers' to refuse: the attention part asks once, at load, and raises instead of rotating wrongly."""
    from mini_rsglang_b200 import InvalidRequest
    from mini_rsglang_b200.parts import PositionEncoding, Rotation

    class Odd(PositionEncoding):
        def __init__(self, prefix, head_dim, rotary_dim, pairing, magnitude):
            super().__init__(prefix)
            self.args = (int(rotary_dim), pairing, float(magnitude))

        def rotation(self):
            return Rotation(torch.ones(self.args[0] // 2, device=DEV), *self.args)

    POSITION_ENCODINGS.register("odd_rotation", Odd, replace=True)
    try:
        width, nq, nkv, d = 40, 2, 1, 16
        for params, word in (({"rotary_dim": 8, "pairing": "split_half", "magnitude": 1.0}, "whole heads"),
                             ({"rotary_dim": 16, "pairing": "interleaved", "magnitude": 1.0}, "pairing"),
                             ({"rotary_dim": 16, "pairing": "split_half", "magnitude": 1.3}, "scaled")):
            mixer = MIXERS.build(PartSpec("gqa_attention", {"width": width, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d,
                                                            "position": PartSpec("odd_rotation", dict(params, head_dim=d))}), "a.self_attn")
            weights = {k: v.to(DEV) for k, v in attention_weights(width, nq, nkv, d, 3).items() if "norm" not in k}
            with pytest.raises(InvalidRequest, match=word):
                mixer.bind(weights, runtime(torch.float32))
    finally:
        POSITION_ENCODINGS.entries.pop("odd_rotation", None)


def test_rotary_part_makes_a_steps_cosines_and_sines_once():
    """Layers with the same frequencies share one table of a step; others get their own; a context without a place for
    shared things gets a fresh table every time."""
    from types import SimpleNamespace

    def rope(d, theta):
        part = POSITION_ENCODINGS.build(PartSpec("rope", {"head_dim": d, "theta": theta}), "p")
        part.bind({}, runtime(torch.float32))
        return part

    first, second, other = rope(128, 1e6), rope(128, 1e6), rope(128, 1e4)
    positions = torch.tensor([0, 1, 5, 4000, 39999], dtype=torch.int32, device=DEV)
    ctx = SimpleNamespace(positions=positions, shared={})
    table = first.rotations(ctx)
    assert second.rotations(ctx) is table and other.rotations(ctx) is not table and len(ctx.shared) == 2
    angles = (positions.float().cpu()[:, None] * P.rope_inverse_frequencies(128, 1e6)[None, :].float()).double()     # float32 products
    close(table[..., 0], torch.cos(angles), torch.float32, "cosines")
    close(table[..., 1], torch.sin(angles), torch.float32, "sines")
    bare = SimpleNamespace(positions=positions)
    assert first.rotations(bare) is not first.rotations(bare)


def attention_weights(width, nq, nkv, d, seed):
    return {"a.self_attn.q_proj.weight": draw((nq * d, width), seed, 0.08),
            "a.self_attn.k_proj.weight": draw((nkv * d, width), seed + 1, 0.08),
            "a.self_attn.v_proj.weight": draw((nkv * d, width), seed + 2, 0.08),
            "a.self_attn.o_proj.weight": draw((width, nq * d), seed + 3, 0.08),
            "a.self_attn.q_norm.weight": draw((d,), seed + 4, 0.1, 1.0),
            "a.self_attn.k_norm.weight": draw((d,), seed + 5, 0.1, 1.0)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,nq,nkv,d,page,tokens", [(40, 5, 5, 16, 4, 23), (88, 6, 2, 64, 8, 70), (56, 4, 1, 80, 16, 33)])
def test_attention_part(dtype, width, nq, nkv, d, page, tokens):
    eps, theta = 2e-6, 30000.0
    head_norm = PartSpec("rmsnorm", {"width": d, "eps": eps})
    spec = PartSpec("gqa_attention", {"width": width, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d,
                                      "q_norm": head_norm, "k_norm": head_norm,
                                      "position": PartSpec("rope", {"head_dim": d, "theta": theta})})
    mixer = MIXERS.build(spec, "a.self_attn")
    weights = attention_weights(width, nq, nkv, d, 10)
    assert sorted(s.name for s in mixer.weight_specs()) == sorted(weights)
    need = mixer.cache_need()
    assert (need.kv_heads, need.head_dim, need.kind) == (nkv, d, "full") and mixer.state_need() is None
    held = {k: v.to(DEV, torch.float32 if v.dim() == 1 else dtype) for k, v in weights.items()}
    mixer.bind(held, runtime(dtype, page))
    ctx, table = whole_sequence_context(tokens, page)
    pages = int(table.max()) + 1
    cache = CacheEntry(group=0, k=torch.zeros((pages, nkv, page, d), dtype=dtype, device=DEV),
                       v=torch.zeros((pages, nkv, page, d), dtype=dtype, device=DEV))
    h = draw((tokens, width), 20, 1.0).to(dtype)
    got = mixer.forward(h.to(DEV), ctx, cache, True)
    cfg = P.PlainConfig(width, 0, 1, nq, nkv, d, 0, eps, theta, False)
    as_held = {k: v.to(dtype) if v.dim() == 2 else v for k, v in weights.items()}
    want = P.attention_part(P.Arith(None), cfg, as_held, "a", h.double(), torch.arange(tokens))
    close(got, want, dtype, "attention part, whole sequence")
    # the second half again, from the cache that the first run left (nothing is written)
    half = tokens // 2
    ctx2, _ = whole_sequence_context(tokens - half, page, first_position=half, table=table)
    again = mixer.forward(h[half:].to(DEV), ctx2, cache, False)
    close(again, want[half:], dtype, "attention part, second half from the cache")


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part(dtype):
    width, inner, tokens = 72, 200, 9
    ff = FEED_FORWARDS.build(PartSpec("swiglu", {"width": width, "inner": inner}), "a.mlp")
    weights = {"a.mlp.gate_proj.weight": draw((inner, width), 1, 0.1), "a.mlp.up_proj.weight": draw((inner, width), 2, 0.1),
               "a.mlp.down_proj.weight": draw((width, inner), 3, 0.1)}
    assert sorted(s.name for s in ff.weight_specs()) == sorted(weights)
    ff.bind({k: v.to(DEV, dtype) for k, v in weights.items()}, runtime(dtype))
    h = draw((tokens, width), 4, 1.0).to(dtype)
    want = P.feed_forward_part(P.Arith(None), {k: v.to(dtype) for k, v in weights.items()}, "a", h.double())
    close(ff.forward(h.to(DEV), None), want, dtype, "feed-forward part")
    with pytest.raises(Exception):
        FEED_FORWARDS.build(PartSpec("swiglu", {"width": 8, "inner": 8, "activation": "gelu"}), "x")


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_arrangement(dtype):
    """pre_norm: the stream takes both branches; the second branch's output comes back pending."""
    width, nq, nkv, d, inner, page, tokens, eps, theta = 48, 3, 1, 32, 100, 4, 19, 1e-5, 1e4
    norm = PartSpec("rmsnorm", {"width": width, "eps": eps})
    head_norm = PartSpec("rmsnorm", {"width": d, "eps": eps})
    block = BLOCKS.get("pre_norm")(
        prefix="a", norm1=NORMS.build(norm, "a.input_layernorm"),
        mixer=MIXERS.build(PartSpec("gqa_attention", {
            "width": width, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d, "q_norm": head_norm,
            "k_norm": head_norm, "position": PartSpec("rope", {"head_dim": d, "theta": theta})}), "a.self_attn"),
        norm2=NORMS.build(norm, "a.post_attention_layernorm"),
        feed_forward=FEED_FORWARDS.build(PartSpec("swiglu", {"width": width, "inner": inner}), "a.mlp"))
    weights = attention_weights(width, nq, nkv, d, 30)
    weights.update({"a.mlp.gate_proj.weight": draw((inner, width), 40, 0.1),
                    "a.mlp.up_proj.weight": draw((inner, width), 41, 0.1),
                    "a.mlp.down_proj.weight": draw((width, inner), 42, 0.1),
                    "a.input_layernorm.weight": draw((width,), 43, 0.1, 1.0),
                    "a.post_attention_layernorm.weight": draw((width,), 44, 0.1, 1.0)})
    assert sorted(s.name for s in block.weight_specs()) == sorted(weights)
    block.bind({k: v.to(DEV, torch.float32 if v.dim() == 1 else dtype) for k, v in weights.items()}, runtime(dtype, page))
    ctx, table = whole_sequence_context(tokens, page)
    pages = int(table.max()) + 1
    cache = CacheEntry(group=0, k=torch.zeros((pages, nkv, page, d), dtype=dtype, device=DEV),
                       v=torch.zeros((pages, nkv, page, d), dtype=dtype, device=DEV))
    x = draw((tokens, width), 50, 1.0)
    stream = x.clone().to(DEV)
    pending = block.forward(stream, None, ctx, cache, True)
    cfg = P.PlainConfig(width, inner, 1, nq, nkv, d, 0, eps, theta, False)
    as_held = {k.replace("a.", "model.layers.0.", 1): (v.to(dtype) if v.dim() == 2 else v) for k, v in weights.items()}
    want = P.block(P.Arith(None), cfg, as_held, 0, x.double(), torch.arange(tokens))
    close(stream.double().cpu() + pending.double().cpu(), want, dtype, "block output = stream + pending")


def test_norms_ride_on_the_products_of_few_rows(monkeypatch):
    """With few rows in bfloat16 the last product of a branch adds to the stream and hands the norm after it
    to the next product (`Prenormed`): the same block output as the plain implementation and as the path
    with the norm's own kernel; a part that does not take a `Prenormed` gets the finished rows."""
    from mini_rsglang_b200 import kernels
    from mini_rsglang_b200.parts.base import Prenormed, plain
    dtype = torch.bfloat16
    width, nq, nkv, d, inner, page, tokens, eps, theta = 136, 2, 1, 128, 192, 4, 6, 1e-5, 1e4
    norm = PartSpec("rmsnorm", {"width": width, "eps": eps})
    head_norm = PartSpec("rmsnorm", {"width": d, "eps": eps})

    def build():
        block = BLOCKS.get("pre_norm")(
            prefix="a", norm1=NORMS.build(norm, "a.input_layernorm"),
            mixer=MIXERS.build(PartSpec("gqa_attention", {
                "width": width, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d, "q_norm": head_norm,
                "k_norm": head_norm, "position": PartSpec("rope", {"head_dim": d, "theta": theta})}), "a.self_attn"),
            norm2=NORMS.build(norm, "a.post_attention_layernorm"),
            feed_forward=FEED_FORWARDS.build(PartSpec("swiglu", {"width": width, "inner": inner}), "a.mlp"))
        block.bind({k: v.to(DEV, torch.float32 if v.dim() == 1 else dtype) for k, v in weights.items()}, runtime(dtype, page))
        return block

    weights = attention_weights(width, nq, nkv, d, 31)
    weights.update({"a.mlp.gate_proj.weight": draw((inner, width), 40, 0.1),
                    "a.mlp.up_proj.weight": draw((inner, width), 41, 0.1),
                    "a.mlp.down_proj.weight": draw((width, inner), 42, 0.1),
                    "a.input_layernorm.weight": draw((width,), 43, 0.1, 1.0),
                    "a.post_attention_layernorm.weight": draw((width,), 44, 0.1, 1.0)})
    after = NORMS.build(norm, "after")
    after.bind({"after.weight": draw((width,), 45, 0.1, 1.0).to(DEV)}, runtime(dtype, page))
    x = draw((tokens, width), 50, 1.0)
    cfg = P.PlainConfig(width, inner, 1, nq, nkv, d, 0, eps, theta, False)
    as_held = {k.replace("a.", "model.layers.0.", 1): (v.to(dtype) if v.dim() == 2 else v) for k, v in weights.items()}
    want = P.block(P.Arith(None), cfg, as_held, 0, x.double(), torch.arange(tokens))

    def run(block):
        ctx, table = whole_sequence_context(tokens, page)
        pages = int(table.max()) + 1
        cache = CacheEntry(group=0, k=torch.zeros((pages, nkv, page, d), dtype=dtype, device=DEV),
                           v=torch.zeros((pages, nkv, page, d), dtype=dtype, device=DEV))
        stream = x.clone().to(DEV)
        norms = []
        real = kernels.add_rmsnorm
        monkeypatch.setattr(kernels, "add_rmsnorm", lambda *a, **k: (norms.append(1), real(*a, **k))[1])
        pending = block.forward(stream, None, ctx, cache, True, next_norm=after)
        monkeypatch.setattr(kernels, "add_rmsnorm", real)
        return stream, pending, len(norms), cache

    stream, pending, norm_launches, cache = run(build())
    assert isinstance(pending, Prenormed) and pending.norm is after and norm_launches == 1      # only the block's first norm
    close(stream.double().cpu(), want, dtype, "the stream holds the block's output")
    sums = pending.square_sums[:, :tokens].sum(0).double().cpu()
    assert ((sums - (stream.double().cpu() ** 2).sum(1)).abs() / sums).max().item() < 1e-5
    close(pending.scaled.double().cpu(), stream.double().cpu() * after.weight.double().cpu(), dtype, "stream times the next weights")
    finished = plain(pending)                                                                 # what a part that takes no Prenormed gets
    close(finished.double().cpu(), P.rms_norm(P.Arith(None), want, after.weight.cpu(), eps), dtype, "finished rows")
    assert after.add_norm(stream, pending) is pending
    # the same block through the norms' own kernels
    monkeypatch.setattr(kernels, "GEMM_TC_BEST_ROWS", 0)
    stream2, pending2, norm_launches2, cache2 = run(build())
    assert isinstance(pending2, torch.Tensor) and norm_launches2 == 2
    close(stream2.double().cpu() + pending2.double().cpu(), want, dtype, "with the norms' own kernels")
    close(cache.k.double().cpu(), cache2.k.double().cpu(), dtype, "keys in the cache")


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    vocab, width = 333, 40
    table = draw((vocab, width), 1, 0.5).to(dtype)
    emb = TokenEmbedding("e", vocab, width)
    emb.bind({"e.weight": table.to(DEV)}, runtime(dtype))
    ctx, _ = whole_sequence_context(5, 4)
    ctx.token_ids = torch.tensor([332, 0, 7, 7, 100], dtype=torch.int32, device=DEV)
    stream = emb.forward(ctx)
    assert stream.dtype is torch.float32
    assert torch.equal(stream.cpu(), table.float()[[332, 0, 7, 7, 100]])
    tied = OutputHead("lm_head", vocab, width, tied_to="e.weight")
    assert tied.weight_specs() == []
    tied.bind({"e.weight": table.to(DEV)}, runtime(dtype))
    hidden = draw((3, width), 2, 1.0).to(dtype)
    logits = tied.forward(hidden.to(DEV))
    assert logits.dtype is torch.float32
    # the inputs are exact in either dtype and the output is not rounded: only the order of the sum differs
    close(logits, hidden.double() @ table.double().T, torch.float32, "head logits keep 32 bits")
