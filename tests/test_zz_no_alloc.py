"""The split-attention entry point that allocates nothing, called the way a host without an
allocator calls it: through its exported C symbol, with raw pointers and a stream.  Such a host
(one that owns the whole device heap itself, or must not stall on an allocation) passes inputs and
output only; the scratch between the two launches is the library's own fixed array.  The test
checks the result against the engine's ordinary entry point, which takes scratch from the caller,
and against the attention formula written out with plain tensor operations, on two calls in a row
(the array keeps the first call's contents); that the device's free memory is the same before and
after a call (the driver's own count, which a cudaMalloc inside the library would move); and that
a call too large for the fixed array is refused.  This file is collected last on purpose."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def build_case(seed, nq=8, nkv=2, d=64, page=16, contexts=(700, 333, 64, 1)):
    from mini_rsglang_b200 import kernels
    g = torch.Generator().manual_seed(seed)
    dev = "cuda:0"
    group = nq // nkv
    per_tile = 16 // group
    pages_needed = sum(-(-(c + per_tile) // page) for c in contexts) + 2
    order = torch.randperm(pages_needed, generator=g).tolist()
    kc = torch.randn(pages_needed, nkv, page, d, generator=g).bfloat16().to(dev)
    vc = torch.randn(pages_needed, nkv, page, d, generator=g).bfloat16().to(dev)
    width = max(-(-(c + per_tile) // page) for c in contexts)
    table = torch.full((len(contexts), width), -1, dtype=torch.int32)
    tiles, positions, row = [], [], 0
    for i, c in enumerate(contexts):
        n = min(per_tile, 1 + i)                         # one to a few new tokens per request
        for lp in range(-(-(c + n) // page)):
            table[i, lp] = order.pop()
        tiles.append((i, row, n, 0))
        positions += list(range(c, c + n))
        row += n
    q = torch.randn(row, nq * d, generator=g).bfloat16().to(dev)
    return dict(lib=kernels.attention_mma_library(d), kernels=kernels, q=q, kc=kc, vc=vc,
                positions=torch.tensor(positions, dtype=torch.int32, device=dev), table=table.to(dev),
                tiles=torch.tensor(tiles, dtype=torch.int32, device=dev), nq=nq, nkv=nkv, d=d, page=page)


def formula(case):
    """softmax(q . k / sqrt(d)) . v over the keys of each request up to the query's position, read through
    the block table, in float64."""
    q, kc, vc = case["q"].double().cpu(), case["kc"].double().cpu(), case["vc"].double().cpu()
    table, positions = case["table"].cpu(), case["positions"].cpu().tolist()
    nq, nkv, d, page = case["nq"], case["nkv"], case["d"], case["page"]
    out = torch.zeros_like(q)
    for seq, first, tokens, _ in case["tiles"].cpu().tolist():
        for row in range(first, first + tokens):
            keys = positions[row] + 1
            pages = table[seq, : -(-keys // page)].long()
            for head in range(nq):
                g = head // (nq // nkv)
                k = kc[pages, g].reshape(-1, d)[:keys]
                v = vc[pages, g].reshape(-1, d)[:keys]
                p = torch.softmax(k @ q[row, head * d:(head + 1) * d] / d ** 0.5, dim=0)
                out[row, head * d:(head + 1) * d] = p @ v
    return out


def call_static(case, splits, out):
    lib = case["lib"]
    fn = lib.mrs_attention_mma_keys_mode_static_scratch
    vp, ci = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [vp, vp, vp, vp, vp, ci, vp, ci, vp, ci, ci, ci, ctypes.c_float, ci, ci, vp]
    fn.restype = ci
    return fn(case["q"].data_ptr(), case["kc"].data_ptr(), case["vc"].data_ptr(), case["positions"].data_ptr(),
              case["table"].data_ptr(), case["table"].shape[1], case["tiles"].data_ptr(), case["tiles"].shape[0],
              out.data_ptr(), case["nq"], case["nkv"], case["page"], 1.0 / case["d"] ** 0.5, 0, splits,
              torch.cuda.current_stream().cuda_stream)


def test_static_scratch_entry_matches_the_ordinary_one_twice_in_a_row():
    for call, (seed, splits) in enumerate([(1, 5), (2, 3)]):
        case = build_case(seed)
        k = case["kernels"]
        want = torch.zeros_like(case["q"])
        k.attention_mma_keys(case["q"], case["kc"], case["vc"], case["positions"], case["table"], case["tiles"], want,
                             case["nq"], case["nkv"], case["d"], 0, splits)
        got = torch.zeros_like(case["q"])
        exact = formula(case)
        if call == 0:                # the first call on the device also looks up the array's address
            assert call_static(case, splits, torch.zeros_like(case["q"])) == 0
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]           # the driver's count of free bytes on the device
        code = call_static(case, splits, got)
        assert code == 0, f"entry point returned {code}"
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
        scale = max(1.0, want.float().abs().max().item())
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 2 ** -7 * scale, f"call {call}: max error {err} against the ordinary entry point"
        err = (got.double().cpu() - exact).abs().max().item()
        assert err <= 2 ** -7 * scale, f"call {call}: max error {err} against the formula"
        assert got.float().abs().max().item() > 0


def test_static_scratch_entry_refuses_what_does_not_fit():
    case = build_case(3)
    lib = case["lib"]
    lib.mrs_attention_mma_error_string.argtypes = [ctypes.c_int]
    lib.mrs_attention_mma_error_string.restype = ctypes.c_char_p
    out = torch.full_like(case["q"], 7.0)
    # 4 tiles * 2 heads * splits * 16 * 66 floats > 4 Mi floats  <=>  splits > 496
    code = call_static(case, 600, out)
    torch.cuda.synchronize()
    assert code == -3 and b"scratch" in lib.mrs_attention_mma_error_string(code)
    assert (out == 7.0).all()                       # nothing was launched
    assert call_static(case, 400, out) == 0
    torch.cuda.synchronize()
