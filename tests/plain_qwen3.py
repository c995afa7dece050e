"""Plain, slow Qwen3-dense implementation used only by the tests.

It rests on the formulas of the reference's source (mirthfulLee/mini-rsglang), not on a run
of it: the reference's model code is Rust over a CUDA backend and cannot be imported or
compiled on a CPU-only machine without a Rust toolchain.  Every function cites the lines it
restates.  What can be compiled of the reference here is compared once: its one CUDA source
(crates/kernels/src/ops.cu) runs on the CPU through small shims.  The kernels that compute one
element a thread (`add`, `rope`, `swiglu`, `embedding`) run thread by thread
(`tests/golden/make_golden.py`); the kernels that work a block together (`rms`, `attention`,
`argmax`) run as one fiber a thread, and a whole two-layer forward pass is put together from those
kernels in the order of the reference's Rust source (`tests/golden/make_model_golden.py`).  The
bfloat16 mode below gives the same bits as all of them (`tests/test_plain.py`).  Whole sequences, no cache, no batching, one function per part; the functions compute
where their tensors lie (the CPU, except for one test of real sizes that gives them tensors on the GPU so
that float64 products of that size take seconds).  Nothing here is
imported by the engine and nothing of the engine is imported here (weights are read with
the `safetensors` package, the engine has a reader of its own).

Two modes:
  * exact  (`rounding=None`): all arithmetic in float64, no intermediate rounding: the
    formulas of the reference with every bf16 rounding removed.  This is the oracle for the
    engine's float32 path and, under a wider gate, for its bfloat16 path.
  * bf16   (`rounding="bf16"`): float32 arithmetic with a round-to-nearest-even to bfloat16
    at every place where the reference's kernels round (`b(...)` in ops.cu).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass

import torch


# --------------------------------------------------------------------------------------
# configuration and weights
# --------------------------------------------------------------------------------------
@dataclass
class PlainConfig:
    """The keys of config.json that the formulas need (crates/models/src/config.rs:8-47)."""

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool

    @staticmethod
    def load(folder: str) -> "PlainConfig":
        with open(os.path.join(folder, "config.json")) as f:
            raw = json.load(f)
        theta = raw.get("rope_theta")
        if theta is None:
            theta = raw["rope_parameters"]["rope_theta"]
        return PlainConfig(
            hidden_size=raw["hidden_size"],
            intermediate_size=raw["intermediate_size"],
            num_hidden_layers=raw["num_hidden_layers"],
            num_attention_heads=raw["num_attention_heads"],
            num_key_value_heads=raw["num_key_value_heads"],
            head_dim=raw["head_dim"],
            vocab_size=raw["vocab_size"],
            rms_norm_eps=raw["rms_norm_eps"],
            rope_theta=theta,
            tie_word_embeddings=raw["tie_word_embeddings"],
        )


def load_plain_weights(folder: str) -> dict[str, torch.Tensor]:
    """All tensors of model.safetensors by name (crates/models/src/weights.rs:40-66)."""
    from safetensors.torch import load_file

    return load_file(os.path.join(folder, "model.safetensors"))


class Arith:
    """Where the reference rounds to bf16, and in which precision the rest is computed."""

    def __init__(self, rounding: str | None):
        assert rounding in (None, "bf16")
        self.rounding = rounding
        self.dtype = torch.float64 if rounding is None else torch.float32

    def r(self, x: torch.Tensor) -> torch.Tensor:
        if self.rounding is None:
            return x
        return x.to(torch.bfloat16).to(torch.float32)

    def w(self, t: torch.Tensor) -> torch.Tensor:
        """A weight as the path sees it (bf16 path: narrowed on load, weights.rs:189-227)."""
        if self.rounding is None:
            return t.to(torch.float64)
        return t.to(torch.bfloat16).to(torch.float32)


# --------------------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------------------
def embedding(ar: Arith, table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """x[t,:] = E[ids[t],:], no scaling (crates/kernels/src/ops.cu:15-18)."""
    return ar.w(table)[ids.long()]


def rms_norm(ar: Arith, x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = r(r(x * rsqrt(mean(x^2) + eps)) * w) over the last axis (ops.cu:66-78)."""
    s = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return ar.r(ar.r(x * s) * ar.w(weight))


def linear(ar: Arith, x: torch.Tensor, weight: torch.Tensor, round_out: bool = True) -> torch.Tensor:
    """y = r(x . W^T), W stored [out, in], no bias (crates/kernels/src/lib.rs:298-321);
    the logits keep 32-bit (lib.rs:785-797)."""
    y = x @ ar.w(weight).T
    return ar.r(y) if round_out else y


def rope_inverse_frequencies(head_dim: int, theta: float) -> torch.Tensor:
    """f_j = 1f32 / f32(theta^(2j/d)) for j in [0, d/2): the power in float64, narrowed to
    float32, the reciprocal in float32 (crates/kernels/src/lib.rs:612-614)."""
    out = []
    for j in range(head_dim // 2):
        power = torch.tensor(float(theta) ** (2 * j / head_dim), dtype=torch.float64).to(torch.float32)
        out.append((torch.tensor(1.0, dtype=torch.float32) / power).to(torch.float64))
    return torch.stack(out)


def rope(ar: Arith, x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Split-half rotary on [T, heads, d] (ops.cu:79-90): pairs (j, j + d/2), angle =
    f32(pos) * f_j, cos and sin rounded, each product rounded, the sum rounded."""
    d = x.shape[-1]
    half = d // 2
    freq = rope_inverse_frequencies(d, theta).to(x.device)
    positions = positions.to(x.device)
    if ar.rounding is None:
        angle = positions.to(torch.float64)[:, None] * freq[None, :]
    else:
        angle = positions.to(torch.float32)[:, None] * freq.to(torch.float32)[None, :]
    c = ar.r(torch.cos(angle)).to(ar.dtype)[:, None, :]
    s = ar.r(torch.sin(angle)).to(ar.dtype)[:, None, :]
    a, z = x[..., :half], x[..., half:]
    first = ar.r(ar.r(a * c) - ar.r(z * s))
    second = ar.r(ar.r(z * c) + ar.r(a * s))
    return torch.cat([first, second], dim=-1)


def causal_attention(ar: Arith, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     window: int = 0) -> torch.Tensor:
    """Causal grouped-query attention of one whole sequence (ops.cu:101-147).
    q [T, nq, d], k and v [T, nkv, d]; query head h reads kv head h // (nq/nkv) (ops.cu:107);
    row t sees keys 0..t (`length = pos + 1`, ops.cu:106), or only the last `window` of them
    (ops.cu:112); score = q.k / sqrt(d) (gpt_oss_ops.rs:45 splits d^-1/4 on both sides);
    softmax in the path's full precision, probabilities unrounded; output rounded once
    (ops.cu:146)."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    out = torch.empty_like(q)
    rows = torch.arange(T, device=q.device)
    mask = rows[None, :] <= rows[:, None]
    if window > 0:
        mask &= rows[None, :] > rows[:, None] - window
    for h in range(nq):
        g = h // group
        scores = (q[:, h, :] @ k[:, g, :].T) / math.sqrt(d)
        scores = scores.masked_fill(~mask, float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        out[:, h, :] = probs @ v[:, g, :]
    return ar.r(out)


def swiglu(ar: Arith, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """a = r(r(g / (1 + exp(-g))) * u) (ops.cu:91-94)."""
    return ar.r(ar.r(gate / (1.0 + torch.exp(-gate))) * up)


def _silent(label: str, tensor: torch.Tensor) -> None:
    pass


def attention_part(ar: Arith, cfg: PlainConfig, w: dict, root: str, n: torch.Tensor,
                   positions: torch.Tensor, observe=_silent, label: str = "") -> torch.Tensor:
    """QKV projection, per-head q/k RMSNorm, rotary, attention, output projection
    (crates/models/src/qwen3.rs:178-202).  `observe` is handed the tensors that the reference's
    observer sees there, under its labels (qwen3.rs:190-201)."""
    T = n.shape[0]
    nq, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    q = linear(ar, n, w[f"{root}.self_attn.q_proj.weight"]).view(T, nq, d)
    k = linear(ar, n, w[f"{root}.self_attn.k_proj.weight"]).view(T, nkv, d)
    v = linear(ar, n, w[f"{root}.self_attn.v_proj.weight"]).view(T, nkv, d)
    observe(f"{label}-q_proj", q.reshape(T, nq * d))
    q = rms_norm(ar, q, w[f"{root}.self_attn.q_norm.weight"], cfg.rms_norm_eps)
    k = rms_norm(ar, k, w[f"{root}.self_attn.k_norm.weight"], cfg.rms_norm_eps)
    observe(f"{label}-q_norm", q.reshape(T, nq * d))
    q = rope(ar, q, positions, cfg.rope_theta)
    k = rope(ar, k, positions, cfg.rope_theta)
    observe(f"{label}-q_rope", q.reshape(T, nq * d))
    observe(f"{label}-k_rope", k.reshape(T, nkv * d))
    observe(f"{label}-v_proj", v.reshape(T, nkv * d))
    attn = causal_attention(ar, q, k, v).reshape(T, nq * d)
    observe(f"{label}-attn", attn)
    return linear(ar, attn, w[f"{root}.self_attn.o_proj.weight"])


def feed_forward_part(ar: Arith, w: dict, root: str, n: torch.Tensor, observe=_silent, label: str = "") -> torch.Tensor:
    """down(swiglu(gate(n), up(n))) (qwen3.rs:239-262, 206-209)."""
    gate = linear(ar, n, w[f"{root}.mlp.gate_proj.weight"])
    up = linear(ar, n, w[f"{root}.mlp.up_proj.weight"])
    activated = swiglu(ar, gate, up)
    observe(f"{label}-swiglu", activated)
    return linear(ar, activated, w[f"{root}.mlp.down_proj.weight"])


def block(ar: Arith, cfg: PlainConfig, w: dict, i: int, x: torch.Tensor,
          positions: torch.Tensor, observe=_silent) -> torch.Tensor:
    """Pre-norm block: x + attn(norm(x)), then + mlp(norm(.)); each sum rounded
    (qwen3.rs:176-225; ops.cu:62-65)."""
    root, label = f"model.layers.{i}", f"layer{i}"
    n = rms_norm(ar, x, w[f"{root}.input_layernorm.weight"], cfg.rms_norm_eps)
    observe(f"{label}-input_norm", n)
    residual = ar.r(x + attention_part(ar, cfg, w, root, n, positions, observe, label))
    n = rms_norm(ar, residual, w[f"{root}.post_attention_layernorm.weight"], cfg.rms_norm_eps)
    out = ar.r(residual + feed_forward_part(ar, w, root, n, observe, label))
    observe(f"{label}-output", out)
    return out


def logits_of_sequence(cfg: PlainConfig, w: dict, tokens, rounding: str | None = None,
                       first_position: int = 0, observe=_silent) -> torch.Tensor:
    """Logits [T, V] at every position of one whole sequence (qwen3.rs:170-236): embedding,
    the blocks in order, the final norm, the head (tied to the embedding when the
    configuration says so, qwen3.rs:234), output unrounded.  `observe(label, tensor)` sees what the
    reference's observer sees, under its labels (qwen3.rs:174-229)."""
    ar = Arith(rounding)
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    positions = torch.arange(first_position, first_position + ids.numel())
    x = embedding(ar, w["model.embed_tokens.weight"], ids).to(ar.dtype)
    observe("embedding", x)
    for i in range(cfg.num_hidden_layers):
        x = block(ar, cfg, w, i, x, positions, observe)
    x = rms_norm(ar, x, w["model.norm.weight"], cfg.rms_norm_eps)
    observe("final_norm", x)
    head = w["model.embed_tokens.weight"] if cfg.tie_word_embeddings else w["lm_head.weight"]
    return linear(ar, x, head, round_out=False)


# --------------------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------------------
def greedy(logits: torch.Tensor) -> int:
    """Largest logit, the smaller id on a tie (ops.cu:152-162)."""
    best = logits.max()
    return int(torch.nonzero(logits == best)[0, 0])


def nucleus_support(logits: torch.Tensor, temperature: float, top_k: int | None,
                    top_p: float) -> tuple[list[int], list[float]]:
    """Ids and unnormalised weights that may be drawn (crates/engine/src/lib.rs:207-244):
    z = logit / T in float64, sorted descending with ties by id, cut to top_k, e = exp(z - max),
    then the shortest prefix whose sum reaches top_p times the sum over the top_k set."""
    z = logits.to(torch.float64) / float(temperature)
    order = sorted(range(z.numel()), key=lambda i: (-float(z[i]), i))
    if top_k is not None:
        order = order[: min(top_k, len(order))]
    top = float(z[order[0]])
    e = [math.exp(float(z[i]) - top) for i in order]
    total = sum(e)
    kept, acc = 0, 0.0
    for value in e:
        acc += value
        kept += 1
        if acc >= top_p * total:
            break
    return order[:kept], e[:kept]


def generate_greedy(cfg: PlainConfig, w: dict, prompt, steps: int,
                    rounding: str | None = None) -> list[int]:
    """Greedy continuation, recomputing the whole sequence for every token."""
    tokens = list(prompt)
    out = []
    for _ in range(steps):
        token = greedy(logits_of_sequence(cfg, w, tokens, rounding)[-1])
        out.append(token)
        tokens.append(token)
    return out
