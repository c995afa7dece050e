"""The plain implementation itself: properties that hold for the formulas whatever the weights."""
import math

import torch
from conftest import TINY_A

import plain_qwen3 as P


def folder_of(model_folders, name):
    return P.PlainConfig.load(model_folders[name]), P.load_plain_weights(model_folders[name])


def test_logits_are_causal(model_folders):
    cfg, w = folder_of(model_folders, "A")
    a = P.logits_of_sequence(cfg, w, [3, 9, 27, 81, 243 % 256, 5])
    b = P.logits_of_sequence(cfg, w, [3, 9, 27, 81, 99, 100])
    assert torch.equal(a[:4], b[:4]) and not torch.equal(a[4], b[4])
    assert a.shape == (6, TINY_A["vocab_size"]) and a.dtype == torch.float64


def test_bf16_mode_is_close_to_exact_and_not_equal(model_folders):
    cfg, w = folder_of(model_folders, "B")
    tokens = list(range(5, 45))
    exact = P.logits_of_sequence(cfg, w, tokens)
    rounded = P.logits_of_sequence(cfg, w, tokens, "bf16").double()
    nrmse = ((exact - rounded).pow(2).mean().sqrt() / exact.pow(2).mean().sqrt()).item()
    assert 0 < nrmse < 0.02


def test_rope_is_a_rotation_and_position_zero_is_identity():
    ar = P.Arith(None)
    x = torch.randn(5, 3, 32, dtype=torch.float64)
    y = P.rope(ar, x, torch.arange(5), 1e6)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    assert torch.equal(y[0], x[0])
    f = P.rope_inverse_frequencies(32, 1e6)
    assert f[0] == 1.0 and abs(f[1].item() - 1e6 ** (-2 / 32)) < 1e-7
    # pairing is (j, j + d/2): rotating a basis vector of dimension 0 moves weight to dimension 16
    e = torch.zeros(1, 1, 32, dtype=torch.float64)
    e[0, 0, 0] = 1.0
    r = P.rope(ar, e, torch.tensor([1]), 1e6)
    assert abs(r[0, 0, 0].item() - math.cos(1.0)) < 1e-12 and abs(r[0, 0, 16].item() - math.sin(1.0)) < 1e-12


def test_attention_of_one_dominant_key_returns_its_value_and_respects_the_window():
    ar = P.Arith(None)
    T, d = 40, 16
    q = torch.zeros(T, 2, d, dtype=torch.float64)
    k = torch.zeros(T, 1, d, dtype=torch.float64)
    v = torch.randn(T, 1, d, dtype=torch.float64)
    q[:, :, 0] = 100.0
    k[7, 0, 0] = 100.0
    out = P.causal_attention(ar, q, k, v)
    assert torch.allclose(out[20, 1], v[7, 0]) and torch.allclose(out[7, 0], v[7, 0])
    assert torch.allclose(out[3, 0], v[:4, 0].mean(dim=0))           # before the key exists: uniform
    windowed = P.causal_attention(ar, q, k, v, window=5)
    assert torch.allclose(windowed[11, 0], v[7, 0]) and torch.allclose(windowed[12, 0], v[8:13, 0].mean(dim=0))


def test_greedy_takes_the_smaller_id_on_a_tie_and_nucleus_support():
    assert P.greedy(torch.tensor([0.0, 2.0, 2.0, 1.0])) == 1
    ids, weights = P.nucleus_support(torch.tensor([0.0, 2.0, 1.0]), 1.0, 2, 0.9)
    assert ids == [1, 2]
    ids, _ = P.nucleus_support(torch.tensor([0.0, 2.0, 1.0]), 1.0, 2, 0.01)
    assert ids == [1]
    ids, _ = P.nucleus_support(torch.tensor([1.0, 1.0, 1.0, 1.0]), 1.0, None, 0.5)
    assert ids == [0, 1]


def test_generation_is_deterministic(model_folders):
    cfg, w = folder_of(model_folders, "A")
    a = P.generate_greedy(cfg, w, [1, 2, 3], 4)
    assert a == P.generate_greedy(cfg, w, [1, 2, 3], 4) and len(a) == 4


# ---------------------------------------------------------------------------------------------
# against the reference's own kernels, compiled for the CPU (tests/golden/make_golden.py)
# ---------------------------------------------------------------------------------------------
def _golden():
    import os

    import numpy as np

    data = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "elementwise.npz"))

    def bf16(name):
        return (torch.from_numpy(data[name].astype(np.int32)) << 16).view(torch.float32)      # bfloat16 bits -> float32

    return data, bf16


def _bits(x: torch.Tensor) -> torch.Tensor:
    """bfloat16 bit patterns of float32 values that are exact in bfloat16."""
    assert torch.equal(x.to(torch.bfloat16).to(torch.float32), x)
    return (x.contiguous().view(torch.int32) >> 16) & 0xFFFF


def test_bf16_mode_rounds_where_the_reference_s_kernels_round():
    """`add`, `swiglu`, `rope` and `embedding` of crates/kernels/src/ops.cu, run thread by thread on the CPU,
    against the plain implementation in bfloat16 mode: the same bits."""
    import numpy as np

    data, bf16 = _golden()
    ar = P.Arith("bf16")
    x, y = bf16("x"), bf16("y")
    want = lambda name: torch.from_numpy(data[name].astype(np.int32))      # noqa: E731
    assert torch.equal(_bits(ar.r(x + y)), want("add"))                    # the residual sum of `block` (ops.cu:62-65)
    assert torch.equal(_bits(P.swiglu(ar, x, y)), want("swiglu"))
    q = bf16("q")
    positions = torch.from_numpy(data["pos"].astype(np.int64))
    assert torch.equal(P.rope_inverse_frequencies(q.shape[-1], float(data["theta"])).to(torch.float32),
                       torch.from_numpy(data["freq"]))
    rotated = P.rope(ar, q, positions, float(data["theta"]))
    mismatches = (_bits(rotated) != want("rope")).sum().item()
    assert mismatches == 0, f"{mismatches} of {rotated.numel()} rotated elements differ"
    table, ids = bf16("table"), torch.from_numpy(data["ids"].astype(np.int64))
    assert torch.equal(_bits(P.embedding(ar, table, ids)), want("embedding"))
    # the layouts that the engine replaces (column split, cache scatter) move bits only
    n, width = x.shape
    assert torch.equal(_bits(x[:, width // 4: width // 4 + width // 2]), want("split"))
    slots = torch.from_numpy(data["slots"].astype(np.int64))
    cache = torch.zeros(2 * n, width)
    cache[slots] = x
    assert torch.equal(_bits(cache), want("kcache"))
