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


# ---------------------------------------------------------------------------------------------
# against the reference's kernels that work a block together, and a whole forward pass made of the
# reference's kernels (tests/golden/make_model_golden.py)
# ---------------------------------------------------------------------------------------------
def _model_golden():
    import os

    import numpy as np

    data = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "model.npz"))

    def bf16(name):
        return (torch.from_numpy(data[name].astype(np.int32)) << 16).view(torch.float32)

    return data, bf16


def _ulps_apart(got: torch.Tensor, want_bits: torch.Tensor) -> torch.Tensor:
    """Distance in bfloat16 steps between values that are exact in bfloat16 (same sign assumed where they differ)."""
    return (_bits(got).to(torch.int64) - want_bits.to(torch.int64)).abs()


def _nearly_the_same_bits(got, want_bits, what, most_differing=0.01):
    """The same bits but for a last-place difference in a few elements: sums that run in another order (the
    reference adds a row's squares thread by thread and warp by warp, a key's products lane by lane) may land on
    the other side of a rounding edge."""
    apart = _ulps_apart(got, want_bits)
    assert apart.max().item() <= 1, f"{what}: {apart.max().item()} bfloat16 steps apart"
    share = (apart > 0).double().mean().item()
    assert share <= most_differing, f"{what}: {share:.4f} of the elements differ in the last place"


def test_rms_norm_is_the_reference_s_rms_kernel():
    import numpy as np
    data, bf16 = _model_golden()
    got = P.rms_norm(P.Arith("bf16"), bf16("rms_x"), bf16("rms_w"), 1e-5)
    _nearly_the_same_bits(got, torch.from_numpy(data["rms_out"].astype(np.int32)), "rms")


def test_attention_is_the_reference_s_attention_kernel_on_a_mixed_batch_over_scrambled_pages():
    """5 tokens that continue a request at position 17 over pages [2, 5] beside a fresh prompt of 37 tokens over pages
    [0, 8, 3] (the reference's operator fixture, crates/kernels/examples/verify_ops.rs:29-47), 6 query heads on 2
    key/value heads; once with every key and once with a window of 7."""
    import numpy as np
    data, bf16 = _model_golden()
    tokens, nq, nkv, d, page, pages, width, window = (int(v) for v in data["att_shape"])
    q = bf16("att_q").view(tokens, nq, d)
    kc, vc = bf16("att_kc").view(pages, page, nkv, d), bf16("att_vc").view(pages, page, nkv, d)
    table, pos, seq = data["att_table"].astype(np.int64), data["att_pos"].astype(np.int64), data["att_seq"].astype(np.int64)
    for name, w in (("att_out", 0), ("att_window_out", window)):
        rows = []
        for s in range(2):
            mine = np.nonzero(seq == s)[0]
            length = int(pos[mine].max()) + 1
            k = kc[torch.from_numpy(table[s])].reshape(-1, nkv, d)[:length]
            v = vc[torch.from_numpy(table[s])].reshape(-1, nkv, d)[:length]
            whole_q = torch.zeros(length, nq, d)
            whole_q[torch.from_numpy(pos[mine])] = q[torch.from_numpy(mine)]
            out = P.causal_attention(P.Arith("bf16"), whole_q, k, v, w)
            rows.append(out[torch.from_numpy(pos[mine])])
        got = torch.cat(rows).reshape(tokens, nq * d)
        _nearly_the_same_bits(got, torch.from_numpy(data[name].astype(np.int32)), name)


def test_greedy_is_the_reference_s_argmax_kernel():
    data, _ = _model_golden()
    logits = torch.from_numpy(data["argmax_x"])
    assert [P.greedy(row) for row in logits] == data["argmax_out"].tolist()
    assert data["argmax_out"].tolist()[:2] == [17, 300]            # a tie takes the smaller id; a late maximum is found


def test_whole_model_is_the_reference_s_kernels_in_the_reference_s_order():
    """A two-layer model run by the reference's own kernels in the order of its `forward_hidden_observed` and `project`
    (crates/models/src/qwen3.rs:160-236) against the plain implementation in bfloat16 mode (nearly the same bits all the
    way: a wrong order, a missing norm or another pairing would differ everywhere) and in exact mode (within the gate of
    the bfloat16 path)."""
    import numpy as np
    data, bf16 = _model_golden()
    layers, hidden, nq, nkv, d, inner, vocab, tokens, _page = (int(v) for v in data["model_shape"])
    cfg = P.PlainConfig(hidden, inner, layers, nq, nkv, d, vocab, float(data["model_eps"]), float(data["model_theta"]), False)
    weights = {name[2:]: bf16(name) for name in data.files if name.startswith("w:")}
    assert torch.equal(P.rope_inverse_frequencies(d, cfg.rope_theta).float(), torch.from_numpy(data["m_freq"]))
    ids = data["m_ids"].astype(np.int64).tolist()
    seen = {}
    got = P.logits_of_sequence(cfg, weights, ids, "bf16", observe=lambda label, t: seen.__setitem__(label, t.clone()))
    for label, name, share in (("layer0-attn", "m_l0_attn", 0.01), ("layer0-output", "m_l0_output", 0.01), ("final_norm", "m_final_norm", 0.01)):
        _nearly_the_same_bits(seen[label], torch.from_numpy(data[name].astype(np.int32)), label, most_differing=share)
    want = torch.from_numpy(data["m_logits"]).double()
    err = (got.double() - want).abs().max().item()
    assert err <= 2 ** -7 * want.abs().max().item(), f"logits of the bfloat16 mode differ by {err}"
    exact = P.logits_of_sequence(cfg, weights, ids)
    nrmse = ((exact - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt()).item()
    assert nrmse <= 0.02, f"exact mode against the reference's kernels: NRMSE {nrmse}"
    assert [P.greedy(row) for row in got] == [P.greedy(row) for row in want.float()]
