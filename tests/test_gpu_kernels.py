"""Each kernel alone against a plain float32/float64 PyTorch statement of the same operation,
at sizes other than the engine's tiny configurations (widths and vocabularies that are no power
of two, head sizes in steps of 16, odd numbers of heads and groups)."""

import pytest
import torch

from mini_rsglang_b200 import BackendError, InvalidRequest, kernels
from mini_rsglang_b200.parts.position import RotaryPosition
from mini_rsglang_b200.sampling import Sampler, SamplingParams, uniform_from_counter
import plain_qwen3 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def close(got, want, dtype, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    if dtype is torch.float32:
        tol = 2e-5 * max(1.0, want.abs().max().item())
    else:
        tol = 2 ** -7 * max(1.0, want.abs().max().item())     # one bfloat16 rounding of the result, with room
    err = (got - want).abs().max().item()
    assert err <= tol, f"{what}: max error {err:.3e} > {tol:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(dtype):
    table = torch.randn(301, 72, device=DEV).to(dtype)
    ids = torch.tensor([0, 300, 5, 5, 17], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 72, device=DEV)
    kernels.embed(table, ids, out)
    assert torch.equal(out, table.float()[ids.long()])


def test_patch_tokens_fills_ids_from_what_another_step_sampled():
    """ids[rows[i]] = sampled[index[i]]; a value that is no token (the sampler's mark of a bad row, or beyond the
    vocabulary) becomes token 0; the other ids stay."""
    ids = torch.arange(100, 140, dtype=torch.int32, device=DEV)
    rows = torch.tensor([3, 0, 39, 17, 20], dtype=torch.int32, device=DEV)
    index = torch.tensor([2, 2, 0, 4, 1], dtype=torch.int32, device=DEV)
    sampled = torch.tensor([7, -1, 299, 5, 300], dtype=torch.int32, device=DEV)
    kernels.patch_tokens(ids, rows, index, sampled, 300)
    want = list(range(100, 140))
    want[3], want[0], want[39], want[17], want[20] = 299, 299, 7, 0, 0
    assert ids.tolist() == want
    big_rows = torch.randperm(5000, device=DEV)[:3000].to(torch.int32)
    big_index = torch.randint(0, 64, (3000,), device=DEV, dtype=torch.int32)
    big_sampled = torch.randint(0, 1000, (64,), device=DEV, dtype=torch.int32)
    big = torch.full((5000,), -5, dtype=torch.int32, device=DEV)
    kernels.patch_tokens(big, big_rows, big_index, big_sampled, 1000)
    expect = torch.full((5000,), -5, dtype=torch.int32, device=DEV)
    expect[big_rows.long()] = big_sampled[big_index.long()]
    assert torch.equal(big, expect)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [72, 75, 1000, 4096, 5120, 16384, 16388])
def test_add_rmsnorm(dtype, width):
    rows = 7
    residual = torch.randn(rows, width, device=DEV)
    delta = torch.randn(rows, width, device=DEV).to(dtype)
    weight = 1 + 0.1 * torch.randn(width, device=DEV)
    eps = 1e-5
    total = residual.double() + delta.double()
    want = total * torch.rsqrt(total.pow(2).mean(-1, keepdim=True) + eps) * weight.double()
    work = residual.clone()
    out = torch.empty(rows, width, device=DEV, dtype=dtype)
    kernels.add_rmsnorm(work, delta, weight, eps, out)
    close(out, want, dtype, "add_rmsnorm")
    close(work, total, torch.float32, "residual written back")
    # picked rows, nothing written back, a row asked for twice
    pick = torch.tensor([6, 0, 6], dtype=torch.int32, device=DEV)
    work = residual.clone()
    out = torch.empty(3, width, device=DEV, dtype=dtype)
    kernels.add_rmsnorm(work, delta, weight, eps, out, rows=pick, write_back=False)
    close(out, want[pick.long()], dtype, "picked rows")
    assert torch.equal(work, residual)
    # no delta
    out = torch.empty(rows, width, device=DEV, dtype=dtype)
    kernels.add_rmsnorm(residual.clone(), None, weight, eps, out)
    x = residual.double()
    close(out, x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight.double(), dtype, "no delta")
    # plain norm of activations
    x = torch.randn(rows, width, device=DEV).to(dtype)
    out = torch.empty_like(x)
    kernels.rmsnorm(x, weight, eps, out)
    xd = x.double()
    close(out, xd * torch.rsqrt(xd.pow(2).mean(-1, keepdim=True) + eps) * weight.double(), dtype, "rmsnorm")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter", [136, 75, 12288])
def test_silu_mul(dtype, inter):
    gate_up = torch.randn(5, 2 * inter, device=DEV).to(dtype) * 3
    out = torch.empty(5, inter, device=DEV, dtype=dtype)
    kernels.silu_mul(gate_up, out)
    g, u = gate_up.double()[:, :inter], gate_up.double()[:, inter:]
    close(out, g / (1 + torch.exp(-g)) * u, dtype, "silu_mul")


@pytest.mark.parametrize("m,n,k", [(1, 7, 5), (33, 100, 72), (64, 64, 16), (130, 301, 257)])
def test_gemm_f32_is_true_float32(m, n, k):
    x = torch.randn(m, k, device=DEV)
    w = torch.randn(n, k, device=DEV)
    out = torch.empty(m, n, device=DEV)
    kernels.gemm_f32(x, w, out)
    want = x.double() @ w.double().T
    close(out, want, torch.float32, "gemm_f32")
    # a product that a tensor-core mode with a shortened mantissa would get wrong by 1e-3
    x = torch.full((1, 8), 1.0 + 2 ** -12, device=DEV)
    w = torch.full((1, 8), 1.0 + 2 ** -12, device=DEV)
    out = torch.empty(1, 1, device=DEV)
    kernels.gemm_f32(x, w, out)
    assert abs(out.item() - 8 * (1 + 2 ** -12) ** 2) < 1e-5
    # a row's result does not depend on the other rows of the batch
    x = torch.randn(70, 72, device=DEV)
    w = torch.randn(50, 72, device=DEV)
    whole, alone = torch.empty(70, 50, device=DEV), torch.empty(1, 50, device=DEV)
    kernels.gemm_f32(x, w, whole)
    kernels.gemm_f32(x[69:70].contiguous(), w, alone)
    assert torch.equal(whole[69:70], alone)


def plain_qk(qkv, positions, q_w, k_w, eps, theta, nq, nkv, d):
    """q and k after head norm and rotation, v untouched, from the plain implementation's parts."""
    ar = P.Arith(None)
    T = qkv.shape[0]
    x = qkv.double().cpu().view(T, nq + 2 * nkv, d)
    q, k, v = x[:, :nq], x[:, nq:nq + nkv], x[:, nq + nkv:]
    if q_w is not None:
        q = P.rms_norm(ar, q, q_w.cpu(), eps)
        k = P.rms_norm(ar, k, k_w.cpu(), eps)
    if theta is not None:
        q = P.rope(ar, q, positions.cpu(), theta)
        k = P.rope(ar, k, positions.cpu(), theta)
    return q, k, v


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page", [(3, 3, 48, 8), (8, 2, 128, 16), (5, 1, 16, 4), (2, 1, 256, 32), (32, 8, 128, 16),
                                           (7, 7, 64, 8), (20, 1, 64, 16)])
def test_qk_norm_rope_store(dtype, nq, nkv, d, page):
    T, pages, eps, theta = 9, 12, 1e-5, 50000.0
    qkv = torch.randn(T, (nq + 2 * nkv) * d, device=DEV).to(dtype)
    positions = torch.tensor([0, 1, 2, 40, 41, 1000, 7, 8, 9], dtype=torch.int32, device=DEV)
    perm = torch.randperm(pages * page)[:T].to(torch.int32).to(DEV)       # scattered, distinct slots
    q_w, k_w = 1 + 0.1 * torch.randn(d, device=DEV), 1 + 0.1 * torch.randn(d, device=DEV)
    inv_freq = RotaryPosition.inverse_frequencies(d, theta).to(DEV)
    assert torch.equal(inv_freq.cpu().double(), P.rope_inverse_frequencies(d, theta))
    q_out = torch.empty(T, nq * d, device=DEV, dtype=dtype)
    kc = torch.zeros(pages, nkv, page, d, device=DEV, dtype=dtype)
    vc = torch.zeros_like(kc)
    kernels.qk_norm_rope_store(qkv, q_out, kc, vc, positions, perm, q_w, k_w, eps, inv_freq, nq, nkv, d, page)
    q, k, v = plain_qk(qkv, positions, q_w, k_w, eps, theta, nq, nkv, d)
    close(q_out.view(T, nq, d), q, dtype, "q")
    slot = perm.long().cpu()
    got_k = kc.cpu()[slot // page, :, slot % page]
    got_v = vc.cpu()[slot // page, :, slot % page]
    close(got_k, k, dtype, "k in the cache")
    assert torch.equal(got_v.double(), v)
    assert kc.count_nonzero().item() <= T * nkv * d                     # nothing else was written
    # no norms, no rotation, no cache: q passes through
    q_only = torch.empty_like(q_out)
    kernels.qk_norm_rope_store(qkv, q_only, None, None, positions, None, None, None, 0.0, None, nq, nkv, d, page)
    assert torch.equal(q_only.view(T, nq, d), qkv.view(T, nq + 2 * nkv, d)[:, :nq])
    with pytest.raises(BackendError, match="refused"):
        kernels.qk_norm_rope_store(torch.zeros(1, 3 * 258, device=DEV), torch.zeros(1, 258, device=DEV), None, None,
                                   positions[:1], None, None, None, 0.0, None, 1, 1, 258, page)


def test_rotation_table_and_many_tokens():
    """The step's table of cosines and sines equals float32 cos and sin of position * frequency, and the kernel that
    reads it gives the same bits with a table handed in as with one it makes itself; 5,000 tokens with 11 heads (the
    warps go around the grid more than once, the last four heads of a token are three), some tokens without a slot."""
    nq, nkv, d, page, eps, theta, tokens = 5, 3, 128, 16, 1e-6, 1e6, 5000
    g = torch.Generator().manual_seed(5)
    positions = torch.randint(0, 40000, (tokens,), generator=g, dtype=torch.int32).to(DEV)
    inv_freq = RotaryPosition.inverse_frequencies(d, theta).to(DEV)
    table = kernels.rotation_table(positions, inv_freq)
    angles = positions.float()[:, None] * inv_freq[None, :]                    # float32 products, as in the kernel
    close(table[..., 0], torch.cos(angles.double()), torch.float32, "cosines")
    close(table[..., 1], torch.sin(angles.double()), torch.float32, "sines")
    qkv = torch.randn(tokens, (nq + 2 * nkv) * d, generator=g).to(torch.bfloat16).to(DEV)
    q_w, k_w = (1 + 0.1 * torch.randn(d, generator=g)).to(DEV), (1 + 0.1 * torch.randn(d, generator=g)).to(DEV)
    pages = tokens // page + 2
    slots = torch.randperm(pages * page, generator=g)[:tokens].to(torch.int32)
    slots[::7] = -1
    outs = []
    for rotations in (None, table):
        q_out = torch.empty(tokens, nq * d, device=DEV, dtype=torch.bfloat16)
        kc = torch.zeros(pages, nkv, page, d, device=DEV, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        kernels.qk_norm_rope_store(qkv, q_out, kc, vc, positions, slots.to(DEV), q_w, k_w, eps, inv_freq, nq, nkv, d, page,
                                   rotations=rotations)
        outs.append((q_out, kc, vc))
    assert all(torch.equal(a, b) for a, b in zip(*outs))
    q, k, v = plain_qk(qkv, positions, q_w, k_w, eps, theta, nq, nkv, d)
    q_out, kc, vc = outs[0]
    close(q_out.view(tokens, nq, d), q, torch.bfloat16, "q")
    keep = (slots >= 0).nonzero().flatten()
    slot = slots[keep].long()
    close(kc.cpu()[slot // page, :, slot % page], k[keep], torch.bfloat16, "k in the cache")
    assert torch.equal(vc.cpu()[slot // page, :, slot % page].double(), v[keep].double())
    assert kc.count_nonzero().item() <= keep.numel() * nkv * d and vc.count_nonzero().item() <= keep.numel() * nkv * d


class PagedCase:
    """Requests with scattered pages; builds the kernel's inputs and the plain answer."""

    def __init__(self, dtype, nq, nkv, d, page, spans, seed=0, window=0):
        # spans: for every request (context already in the cache, new tokens in this step)
        g = torch.Generator().manual_seed(seed)
        self.nq, self.nkv, self.d, self.page, self.window, self.dtype = nq, nkv, d, page, window, dtype
        total_pages = sum(-(-(c + n) // page) for c, n in spans) + 3
        order = torch.randperm(total_pages, generator=g).tolist()
        self.kc = torch.zeros(total_pages, nkv, page, d, dtype=dtype)
        self.vc = torch.zeros_like(self.kc)
        width = max(-(-(c + n) // page) for c, n in spans)
        self.table = torch.full((len(spans), width), -1, dtype=torch.int32)
        q_rows, pos, seq, self.want, self.q_start = [], [], [], [], [0]
        self.ks, self.vs = [], []
        for i, (c, n) in enumerate(spans):
            L = c + n
            k = torch.randn(L, nkv, d, generator=g).to(dtype)
            v = torch.randn(L, nkv, d, generator=g).to(dtype)
            q = torch.randn(n, nq, d, generator=g).to(dtype)
            self.ks.append(k), self.vs.append(v)
            for lp in range(-(-L // page)):
                page_id = order.pop()
                self.table[i, lp] = page_id
                rows = slice(lp * page, min(L, (lp + 1) * page))
                self.kc[page_id, :, :rows.stop - rows.start] = k[rows].transpose(0, 1)
                self.vc[page_id, :, :rows.stop - rows.start] = v[rows].transpose(0, 1)
            q_rows.append(q)
            pos += list(range(c, L))
            seq += [i] * n
            self.q_start.append(self.q_start[-1] + n)
        self.q = torch.cat(q_rows)
        self.positions = torch.tensor(pos, dtype=torch.int32)
        self.seq = torch.tensor(seq, dtype=torch.int32)
        self.spans = spans

    def plain(self):
        ar = P.Arith(None)
        out = []
        for i, (c, n) in enumerate(self.spans):
            L = c + n
            full_q = torch.zeros(L, self.nq, self.d, dtype=torch.float64)
            full_q[c:] = self.q[self.q_start[i]:self.q_start[i + 1]].double()
            o = P.causal_attention(ar, full_q, self.ks[i].double(), self.vs[i].double(), self.window)
            out.append(o[c:])
        return torch.cat(out).reshape(-1, self.nq * self.d)

    def dev(self, t):
        return t.to(DEV)

    def run_simt(self):
        out = torch.empty(self.q.shape[0], self.nq * self.d, device=DEV, dtype=self.dtype)
        kernels.attention_simt(self.dev(self.q.reshape(-1, self.nq * self.d)), self.dev(self.kc), self.dev(self.vc),
                               self.dev(self.positions), self.dev(self.seq), self.dev(self.table), out, self.nq,
                               self.nkv, self.d, self.window)
        return out

    def run_mma(self, mode, splits=1):
        group = self.nq // self.nkv
        per_tile = {"rows": 64}.get(mode, 16) // group
        if mode in ("tc", "tc_shares", "tc_pairs"):          # two tiles of 128 rows, each a whole number of tokens
            per_tile = 2 * (128 // group)
        tiles = []
        for i in range(len(self.spans)):
            first, n = self.q_start[i], self.q_start[i + 1] - self.q_start[i]
            if mode == "tc_pairs":               # the first tile of a request with its last, the second with the last but one, ...
                one = 128 // group
                count = -(-n // one)
                for a in range(count // 2):
                    b = count - 1 - a
                    tiles.append((i, first + a * one, one + min(one, n - b * one), ((b - a - 1) * one) << 16))
                if count % 2:
                    tiles.append((i, first + (count // 2) * one, min(one, n - (count // 2) * one), 0))
                continue
            for s in range(0, n, per_tile):
                if mode == "tc_shares":          # `splits` entries that walk one share of the keys each
                    tiles += [(i, first + s, min(per_tile, n - s), share | splits << 8) for share in range(splits)]
                else:
                    tiles.append((i, first + s, min(per_tile, n - s), 0))
        tiles = torch.tensor(tiles, dtype=torch.int32, device=DEV)
        out = torch.zeros(self.q.shape[0], self.nq * self.d, device=DEV, dtype=self.dtype)
        args = (self.dev(self.q.reshape(-1, self.nq * self.d)), self.dev(self.kc), self.dev(self.vc),
                self.dev(self.positions), self.dev(self.table), tiles, out, self.nq, self.nkv, self.d, self.window)
        if mode == "keys":
            kernels.attention_mma_keys(*args, splits=splits)
        elif mode in ("tc", "tc_shares", "tc_pairs"):
            kernels.attention_prefill_tc(*args, shares=mode == "tc_shares")
            torch.cuda.synchronize()
            kernels.check_device_errors()
        elif mode == "tma":
            kernels.attention_decode_tma(*args, splits=splits)
            torch.cuda.synchronize()
            kernels.check_device_errors()
        else:
            kernels.attention_mma_rows(*args)
        return out


SHAPES = [(3, 3, 48, 8), (8, 2, 128, 16), (6, 1, 32, 4), (4, 2, 16, 16), (2, 1, 256, 32), (5, 5, 80, 16), (12, 2, 64, 64)]
SPANS = [(0, 1), (0, 70), (130, 3), (257, 1), (63, 66), (1, 2), (300, 1)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page", SHAPES)
def test_attention_simt(dtype, nq, nkv, d, page):
    case = PagedCase(dtype, nq, nkv, d, page, SPANS, seed=nq * d)
    close(case.run_simt(), case.plain(), dtype, "attention_simt")


@pytest.mark.parametrize("window", [1, 5, 64, 100])
def test_attention_window_edges(window):
    for dtype in DTYPES:
        case = PagedCase(dtype, 4, 2, 32, 8, [(0, 130), (120, 1), (99, 2), (3, 4)], seed=window, window=window)
        close(case.run_simt(), case.plain(), dtype, f"simt window {window}")
    case = PagedCase(torch.bfloat16, 4, 2, 32, 8, [(0, 130), (120, 1), (99, 2), (3, 4)], seed=window, window=window)
    close(case.run_mma("rows"), case.plain(), torch.bfloat16, f"mma rows window {window}")
    close(case.run_mma("keys", 1), case.plain(), torch.bfloat16, f"mma keys window {window}")
    close(case.run_mma("keys", 3), case.plain(), torch.bfloat16, f"mma keys split window {window}")


@pytest.mark.parametrize("nq,nkv,d,page", SHAPES)
def test_attention_mma_rows_mode(nq, nkv, d, page):
    case = PagedCase(torch.bfloat16, nq, nkv, d, page, SPANS, seed=nq + d)
    close(case.run_mma("rows"), case.plain(), torch.bfloat16, "attention_mma rows")


@pytest.mark.parametrize("splits", [1, 2, 5, 16])
@pytest.mark.parametrize("nq,nkv,d,page", SHAPES)
def test_attention_mma_keys_mode(nq, nkv, d, page, splits):
    case = PagedCase(torch.bfloat16, nq, nkv, d, page, SPANS, seed=nq + d + splits)
    close(case.run_mma("keys", splits), case.plain(), torch.bfloat16, f"attention_mma keys, {splits} splits")


TMA_SHAPES = [(8, 2, 128, 16), (2, 1, 256, 32), (12, 2, 64, 64), (4, 4, 64, 8), (16, 1, 128, 128), (3, 1, 192, 16)]


@pytest.mark.parametrize("splits", [1, 2, 5, 16])
@pytest.mark.parametrize("nq,nkv,d,page", TMA_SHAPES)
def test_attention_decode_tma(nq, nkv, d, page, splits):
    """Head sizes 64 to 256, pages of 8 to 128 rows (a copy of a whole page, and of 64 rows of a
    longer one), groups of 1 to 16 query heads."""
    assert kernels.attention_decode_tma_supported(d, nq // nkv, page)
    case = PagedCase(torch.bfloat16, nq, nkv, d, page, SPANS, seed=nq + d + splits)
    close(case.run_mma("tma", splits), case.plain(), torch.bfloat16, f"attention_decode_tma, {splits} splits")


TC_SHAPES = [(8, 2, 128, 16), (12, 3, 64, 8), (4, 4, 64, 64), (16, 1, 128, 128), (2, 1, 128, 32), (32, 1, 64, 16),
             (10, 2, 128, 16), (3, 1, 64, 8), (14, 2, 128, 32), (48, 1, 64, 16)]      # groups of 5, 3, 7, 48: rows of a tile stay empty
TC_SPANS = [(0, 1), (0, 70), (130, 3), (257, 1), (63, 66), (1, 2), (300, 200), (0, 513), (1000, 37)]


@pytest.mark.parametrize("nq,nkv,d,page", TC_SHAPES)
def test_attention_prefill_tc(nq, nkv, d, page):
    """Head sizes 64 and 128, groups of 1 to 48 query heads (among them groups that do not divide a tile's 128
    rows), pages of 8 to 128 rows; portions of 1 to 513 tokens on contexts up to 1,037: several tiles a request,
    several blocks of keys a tile, blocks that need no mask, the diagonal, and tiles that are not full."""
    assert kernels.attention_prefill_tc_supported(d, nq // nkv, page)
    case = PagedCase(torch.bfloat16, nq, nkv, d, page, TC_SPANS, seed=nq + d)
    close(case.run_mma("tc"), case.plain(), torch.bfloat16, "attention_prefill_tc")


@pytest.mark.parametrize("shares", [2, 3, 7])
@pytest.mark.parametrize("nq,nkv,d,page", [(8, 2, 128, 16), (4, 4, 64, 8), (4, 1, 128, 32), (10, 2, 128, 16)])
def test_attention_prefill_tc_shares_of_the_keys(nq, nkv, d, page, shares):
    """Entries that walk one share of their key blocks each, merged by the second kernel: portions deep in a long
    context, a fresh prompt whose first entries have fewer blocks than shares (empty shares), a tile without
    a block in the last share, a ragged last entry."""
    case = PagedCase(torch.bfloat16, nq, nkv, d, page, [(1000, 70), (0, 300), (130, 3 + 2 * (128 // (nq // nkv))), (2000, 40)], seed=shares)
    close(case.run_mma("tc_shares", shares), case.plain(), torch.bfloat16, f"{shares} shares of the keys")


@pytest.mark.parametrize("nq,nkv,d,page", [(8, 2, 128, 16), (4, 4, 64, 8), (10, 2, 128, 16), (2, 1, 128, 32), (16, 8, 128, 16)])
def test_attention_prefill_tc_tiles_that_are_no_neighbours(nq, nkv, d, page):
    """Entries whose two tiles lie apart in their request (the first tile with the last, and so on inwards): a tile
    that is done after one block beside one that walks a dozen, a last tile that is not full, an odd count whose
    middle tile stands alone, requests of one and two tiles, and cached tokens before the portion."""
    one = 128 // (nq // nkv)
    case = PagedCase(torch.bfloat16, nq, nkv, d, page, [(0, 12 * one), (0, 7 * one + 3), (300, 5 * one - 1), (0, one), (64, 2 * one), (0, 3)], seed=nq)
    close(case.run_mma("tc_pairs"), case.plain(), torch.bfloat16, "tiles that are no neighbours")
    assert torch.equal(case.run_mma("tc_pairs"), case.run_mma("tc"))          # a row's walk is the same whoever shares its CTA


def test_attention_prefill_tc_rescales_when_the_maximum_grows():
    """Keys whose scores rise block after block by far more than 2^8: the accumulator in tensor
    memory is rescaled again and again; then keys that fall: it is not."""
    nq, nkv, d, page = 4, 2, 64, 16
    for rising in (True, False):
        case = PagedCase(torch.bfloat16, nq, nkv, d, page, [(0, 600)], seed=3)
        case.q.mul_(0.05)
        case.q[:, :, 5] = 4.0
        ramp = torch.arange(600, dtype=torch.float32) / 600 * 24 - 12          # scores from -6 to +6 (in natural units)
        case.ks[0].mul_(0.05)
        case.ks[0][:, :, 5] = (ramp if rising else -ramp).to(torch.bfloat16)[:, None] * (d ** 0.5) / 4.0 / 2
        for lp in range(-(-600 // page)):
            rows = slice(lp * page, min(600, (lp + 1) * page))
            case.kc[case.table[0, lp], :, :rows.stop - rows.start] = case.ks[0][rows].transpose(0, 1)
        close(case.run_mma("tc"), case.plain(), torch.bfloat16, f"prefill_tc, scores {'rising' if rising else 'falling'}")


@pytest.mark.parametrize("window", [1, 5, 64, 100, 300])
def test_attention_prefill_tc_window_edges(window):
    case = PagedCase(torch.bfloat16, 4, 2, 64, 8, [(0, 330), (120, 40), (99, 2), (3, 4)], seed=window, window=window)
    close(case.run_mma("tc"), case.plain(), torch.bfloat16, f"prefill_tc window {window}")


@pytest.mark.parametrize("window", [1, 5, 64, 100])
def test_attention_decode_tma_window_edges(window):
    case = PagedCase(torch.bfloat16, 4, 2, 64, 8, [(0, 130), (120, 1), (99, 2), (3, 4)], seed=window, window=window)
    close(case.run_mma("tma", 1), case.plain(), torch.bfloat16, f"tma window {window}")
    close(case.run_mma("tma", 3), case.plain(), torch.bfloat16, f"tma split window {window}")
    # pages that the window has passed are gone from the table: the kernel must not need them
    table = case.table.clone()
    for i, (c, n) in enumerate(case.spans):
        passed = max(0, c - window + 1) // case.page
        case.table[i, :passed] = -1
    close(case.run_mma("tma", 2), case.plain(), torch.bfloat16, f"tma window {window}, passed pages given back")
    case.table = table


@pytest.mark.parametrize("runner", ["simt32", "simt16", "rows", "keys1", "keys7", "tma1", "tma7", "tc"])
def test_one_far_key_among_hundreds(runner):
    """One key far back scores far above the rest: the output must be that key's value row, so a
    kernel that skips, repeats or misplaces a block of keys cannot pass."""
    dtype = torch.float32 if runner == "simt32" else torch.bfloat16
    nq, nkv, d, page = 4, 2, 64, 16
    for far in (0, 15, 16, 63, 64, 200, 511, 689):
        case = PagedCase(dtype, nq, nkv, d, page, [(700, 1), (690, 12)], seed=far)
        for i in range(2):
            case.ks[i].mul_(0.01)
            case.ks[i][far] = 0
            case.ks[i][far, :, 3] = 16.0
        case.q.mul_(0.01)
        case.q[:, :, 3] = 16.0
        # rebuild the cache pages from the edited keys
        for i, (c, n) in enumerate(case.spans):
            L = c + n
            for lp in range(-(-L // page)):
                rows = slice(lp * page, min(L, (lp + 1) * page))
                case.kc[case.table[i, lp], :, :rows.stop - rows.start] = case.ks[i][rows].transpose(0, 1)
        got = {"simt32": case.run_simt, "simt16": case.run_simt, "rows": lambda: case.run_mma("rows"),
               "keys1": lambda: case.run_mma("keys", 1), "keys7": lambda: case.run_mma("keys", 7),
               "tma1": lambda: case.run_mma("tma", 1), "tma7": lambda: case.run_mma("tma", 7),
               "tc": lambda: case.run_mma("tc")}[runner]()
        want_rows = torch.cat([case.vs[0][far].reshape(1, -1).repeat(1, 1)] +
                              [case.vs[1][far].reshape(1, -1)] * 12).double()
        want = want_rows.view(13, nkv, 1, d).expand(13, nkv, nq // nkv, d).reshape(13, nq * d)
        close(got, want, dtype, f"{runner}, far key at {far}")
        close(got, case.plain(), dtype, f"{runner} vs plain, far key at {far}")


@pytest.mark.parametrize("runner", ["simt16", "tma1", "tma16", "tma7", "tma15", "tma32", "tc"])
def test_one_far_key_among_tens_of_thousands(runner):
    """The same at a context of 40,000 tokens with heads of 128 (block tables of 2,500 pages, scattered): a decoded
    token and a portion of a prompt find one key at the start, in the middle and near the end.  The shares of the
    keys as one cluster (16) and as counts that are no cluster and meet through memory (7, 15, 32: what the plan
    takes for few requests with long contexts)."""
    dtype = torch.bfloat16
    nq, nkv, d, page = 8, 2, 128, 16
    case = PagedCase(dtype, nq, nkv, d, page, [(39990, 1), (39000, 70)], seed=9)
    case.q.mul_(0.01)
    case.q[:, :, 5] = 16.0
    keys_as_drawn = [k.clone() for k in case.ks]
    for far in (0, 17, 20000, 38999):
        for i, (c, n) in enumerate(case.spans):
            case.ks[i] = keys_as_drawn[i] * 0.01
            case.ks[i][far] = 0
            case.ks[i][far, :, 5] = 16.0
            for lp in range(-(-(c + n) // page)):
                rows = slice(lp * page, min(c + n, (lp + 1) * page))
                case.kc[case.table[i, lp], :, :rows.stop - rows.start] = case.ks[i][rows].transpose(0, 1)
        if runner.startswith("tma"):
            got = case.run_mma("tma", int(runner[3:]))
        else:
            got = {"simt16": case.run_simt, "tc": lambda: case.run_mma("tc")}[runner]()
        want_rows = torch.cat([case.vs[0][far].reshape(1, -1)] + [case.vs[1][far].reshape(1, -1)] * 70).double()
        want = want_rows.view(71, nkv, 1, d).expand(71, nkv, nq // nkv, d).reshape(71, nq * d)
        close(got, want, dtype, f"{runner}, far key at {far} of 40,000")


def test_attention_refuses_what_it_cannot_do():
    case = PagedCase(torch.bfloat16, 4, 2, 32, 8, [(0, 4)])
    with pytest.raises(InvalidRequest):
        kernels.attention_simt(case.dev(case.q.reshape(-1, 128)).float(), case.dev(case.kc), case.dev(case.vc),
                               case.dev(case.positions), case.dev(case.seq), case.dev(case.table),
                               torch.empty(4, 128, device=DEV), 4, 2, 32)
    assert not kernels.attention_mma_supported(24, 1) and not kernels.attention_mma_supported(128, 128)
    assert kernels.attention_mma_supported(112, 7)
    assert not kernels.attention_decode_tma_supported(48, 1, 16) and not kernels.attention_decode_tma_supported(128, 4, 4)


# --------------------------------------------------------------------------------- tcgen05 product
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,n,k", [(1, 7, 8), (8, 128, 64), (16, 300, 72), (17, 1000, 1000), (64, 4096, 4096),
                                   (100, 257, 136), (128, 6144, 520), (3, 24576, 4096)])
def test_gemm_tc(m, n, k, out_dtype):
    """Rows up to 128 (every padded size), widths and depths that are no multiples of the tiles,
    one and several ranges of K."""
    g = torch.Generator().manual_seed(m + n + k)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    assert kernels.gemm_tc_supported(x.to(DEV), w.to(DEV))
    out = torch.full((m, n), float("nan"), dtype=out_dtype, device=DEV)
    kernels.gemm_tc(x.to(DEV), w.to(DEV), out)
    torch.cuda.synchronize()
    kernels.check_device_errors()
    close(out, x.double() @ w.double().T, out_dtype, f"gemm_tc {m}x{n}x{k}")


@pytest.mark.parametrize("m,inner,k", [(1, 64, 72), (8, 128, 64), (19, 3072, 1024), (32, 192, 4096), (100, 12288, 520)])
def test_gemm_tc_gated(m, inner, k):
    """silu(x . gate^T) * (x . up^T) out of one product over weights in blocks of 64 gate and 64 up rows;
    the same result as the product followed by the kernel that does it alone."""
    g = torch.Generator().manual_seed(m + inner)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    gate = (torch.randn(inner, k, generator=g) / k ** 0.5 * 2).to(torch.bfloat16)
    up = (torch.randn(inner, k, generator=g) / k ** 0.5 * 2).to(torch.bfloat16)
    mixed = torch.stack([gate.view(-1, 64, k), up.view(-1, 64, k)], dim=1).reshape(2 * inner, k).contiguous()
    out = torch.full((m, inner), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.gemm_tc(x.to(DEV), mixed.to(DEV), out, gated=True)
    torch.cuda.synchronize()
    kernels.check_device_errors()
    gd, ud = x.double() @ gate.double().T, x.double() @ up.double().T
    want = gd / (1 + torch.exp(-gd)) * ud
    close(out, want, torch.bfloat16, f"gated gemm_tc {m}x{inner}x{k}")
    both = torch.cat([gd.unsqueeze(0), ud.unsqueeze(0)])      # the kernel alone on the blocked layout
    blocked = torch.stack([gd.view(m, -1, 64), ud.view(m, -1, 64)], dim=2).reshape(m, 2 * inner).to(torch.bfloat16).to(DEV)
    alone = torch.empty((m, inner), dtype=torch.bfloat16, device=DEV)
    kernels.silu_mul(blocked, alone, 64)
    close(alone, want, torch.bfloat16, "silu_mul on blocks of 64")
    del both


@pytest.mark.parametrize("t,inner,k", [(1, 64, 72), (128, 128, 64), (200, 192, 136), (513, 3072, 1024), (2048, 12288, 4096), (300, 64, 520)])
def test_gemm_gated_rows(t, inner, k):
    """The gated product for many rows (tiles of 128 tokens x 256 weight rows): token counts and widths that end inside
    a tile, a weight matrix of one and a half tiles, a depth that ends inside a block of 64."""
    g = torch.Generator().manual_seed(t + inner)
    x = torch.randn(t, k, generator=g).to(torch.bfloat16)
    gate = (torch.randn(inner, k, generator=g) / k ** 0.5 * 2).to(torch.bfloat16)
    up = (torch.randn(inner, k, generator=g) / k ** 0.5 * 2).to(torch.bfloat16)
    mixed = torch.stack([gate.view(-1, 64, k), up.view(-1, 64, k)], dim=1).reshape(2 * inner, k).contiguous()
    assert kernels.gemm_gated_rows_supported(x.to(DEV), mixed.to(DEV))
    out = torch.full((t, inner), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.gemm_gated_rows(x.to(DEV), mixed.to(DEV), out)
    torch.cuda.synchronize()
    kernels.check_device_errors()
    gd, ud = x.double() @ gate.double().T, x.double() @ up.double().T
    close(out, gd / (1 + torch.exp(-gd)) * ud, torch.bfloat16, f"gated rows {t}x{inner}x{k}")
    assert not kernels.gemm_gated_rows_supported(x.to(DEV), mixed.to(DEV)[:64])          # half a block of gate rows


@pytest.mark.parametrize("m,nq,nkv,k,page", [(1, 2, 1, 64, 8), (8, 32, 8, 4096, 16), (19, 3, 3, 520, 4), (32, 8, 2, 1024, 32)])
def test_gemm_tc_qkv_heads(m, nq, nkv, k, page):
    """The fused q/k/v projection with head norms, rotation and cache write in its epilogue, against the
    plain functions; and against the product followed by the kernel that does the rest alone."""
    d, eps, theta, pages = 128, 1e-6, 1e6, 9
    g = torch.Generator().manual_seed(m + nq + k)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn((nq + 2 * nkv) * d, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    q_w, k_w = 1 + 0.1 * torch.randn(d, generator=g), 1 + 0.1 * torch.randn(d, generator=g)
    positions = torch.randint(0, 3000, (m,), generator=g, dtype=torch.int32)
    slots = torch.randperm(pages * page, generator=g)[:m].to(torch.int32)
    slots[m // 2] = -1 if m > 1 else slots[0]                 # a row that writes nothing
    inv_freq = RotaryPosition.inverse_frequencies(d, theta)
    q_out = torch.full((m, nq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros(pages, nkv, page, d, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    kernels.gemm_tc_qkv_heads(x.to(DEV), w.to(DEV), q_out, kc, vc, positions.to(DEV), slots.to(DEV), q_w.to(DEV), k_w.to(DEV),
                              eps, inv_freq.to(DEV), nq, nkv)
    torch.cuda.synchronize()
    kernels.check_device_errors()
    qkv = (x.double() @ w.double().T).float()                  # the plain functions on the unrounded product
    q, kk, v = plain_qk(qkv.to(DEV), positions.to(DEV), q_w.to(DEV), k_w.to(DEV), eps, theta, nq, nkv, d)
    close(q_out.view(m, nq, d), q, torch.bfloat16, "q")
    keep = (slots >= 0).nonzero().flatten()
    slot = slots[keep].long()
    close(kc.cpu()[slot // page, :, slot % page], kk[keep], torch.bfloat16, "k in the cache")
    close(vc.cpu()[slot // page, :, slot % page], v[keep], torch.bfloat16, "v in the cache")
    assert kc.count_nonzero().item() <= keep.numel() * nkv * d and vc.count_nonzero().item() <= keep.numel() * nkv * d
    # q only: nothing is written without slots
    kc.zero_()
    kernels.gemm_tc_qkv_heads(x.to(DEV), w.to(DEV), q_out, None, None, positions.to(DEV), None, q_w.to(DEV), k_w.to(DEV), eps,
                              inv_freq.to(DEV), nq, nkv)
    close(q_out.view(m, nq, d), q, torch.bfloat16, "q without a cache")
    assert kc.count_nonzero().item() == 0


@pytest.mark.parametrize("m,n,k", [(1, 128, 64), (8, 4096, 4096), (5, 136, 192), (8, 1000, 12288), (19, 520, 1024), (32, 256, 320)])
def test_gemm_tc_adds_to_the_stream_and_prepares_the_next_norm(m, n, k):
    """The product whose epilogue adds to the residual stream: stream += bfloat16(x . w^T), out = stream * the next
    norm's weights, and parts of the rows' sums of squares that add up to the rows' sums of squares."""
    g = torch.Generator().manual_seed(m * n + k)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    stream = 3 * torch.randn(m, n, generator=g)
    next_w = 1 + 0.2 * torch.randn(n, generator=g)
    on_device = stream.clone().to(DEV)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    sums = kernels.gemm_tc(x.to(DEV), w.to(DEV), out, residual=(on_device, next_w.to(DEV)))
    torch.cuda.synchronize()
    kernels.check_device_errors()
    product = (x.double() @ w.double().T)
    want_stream = stream.double() + product
    error = (on_device.cpu().double() - want_stream).abs()              # one bfloat16 rounding of the product, one float32 sum
    assert (error <= 2.0 ** -8 * product.abs() + 1e-5).all(), f"stream: {error.max().item():.3e}"
    close(out, want_stream * next_w.double(), torch.bfloat16, "stream times the next norm's weights")
    assert sums.shape[0] == (n + 127) // 128
    got = sums[:, :m].sum(0).cpu().double()
    exact = (on_device.cpu().double() ** 2).sum(1)                      # of the stream that the kernel wrote
    assert ((got - exact).abs() / exact).max().item() < 1e-5, "sums of squares"


@pytest.mark.parametrize("m", [1, 8, 16, 30])
def test_gemm_tc_more_ranges_for_the_tiles_of_the_last_round(m):
    """A plan of two counts of ranges (the first tiles 2, the tiles behind them 4 or 3), as the library plans a last
    round of units that would fill the GPU partly: plain, gated and adding to the stream, all equal to the same
    product with one count; and the plans of the shapes it was made for."""
    lib = kernels.gemm_tc_library()
    assert lib.mrs_gemm_tc_splits(24576, 4096, 148) == 2 | 3 << 8 | 148 << 16           # gate/up of the 8B shape: 44 tiles in the last round
    assert lib.mrs_gemm_tc_splits(151936, 4096, 148) == 1 | 16 << 8 | 1184 << 16        # the head: 3 tiles
    assert lib.mrs_gemm_tc_splits(4096, 4096, 148) == 4 and lib.mrs_gemm_tc_splits(6144, 4096, 148) == 3
    n, k = 20 * 128 + 72, 1024
    g = torch.Generator().manual_seed(m)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16).to(DEV)
    want = x.double().cpu() @ w.double().cpu().T
    for plan in (2 | 4 << 8 | 12 << 16, 1 | 3 << 8 | 20 << 16, 3 | 2 << 8 | 1 << 16):
        out = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
        kernels.gemm_tc(x, w, out, splits=plan)
        close(out, want, torch.float32, f"plan {plan:#x}")
        stream = (3 * torch.randn(m, n, generator=g)).to(DEV)
        before = stream.clone()
        folded = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
        sums = kernels.gemm_tc(x, w, folded, splits=plan, residual=(stream, torch.ones(n, device=DEV)))
        error = (stream.double().cpu() - before.double().cpu() - want).abs()
        assert (error <= 2.0 ** -8 * want.abs() + 1e-5).all(), f"stream with plan {plan:#x}: {error.max().item():.3e}"
        exact = (stream.double() ** 2).sum(1).cpu()
        assert ((sums[:, :m].sum(0).cpu().double() - exact).abs() / exact).max().item() < 1e-5
    inner = 20 * 64
    mixed = (torch.randn(2 * inner, k, generator=g) / k ** 0.5 * 2).to(torch.bfloat16).to(DEV)
    outs = []
    for plan in (2 | 4 << 8 | 12 << 16, 2):
        out = torch.full((m, inner), float("nan"), dtype=torch.bfloat16, device=DEV)
        kernels.gemm_tc(x, mixed, out, gated=True, splits=plan)
        outs.append(out)
    both = x.double().cpu() @ mixed.double().cpu().T
    gd, ud = both.view(m, -1, 2, 64)[:, :, 0].reshape(m, inner), both.view(m, -1, 2, 64)[:, :, 1].reshape(m, inner)
    close(outs[0], gd / (1 + torch.exp(-gd)) * ud, torch.bfloat16, "gated with two counts of ranges")
    assert torch.equal(outs[0][:, :12 * 64], outs[1][:, :12 * 64])      # the tiles with 2 ranges: the same bits either way
    torch.cuda.synchronize()
    kernels.check_device_errors()


@pytest.mark.parametrize("m,n,k,out_dtype", [(1, 256, 136, torch.float32), (8, 151936 // 8, 4096, torch.float32),
                                            (7, 520, 1024, torch.bfloat16), (40, 384, 512, torch.bfloat16)])
def test_gemm_tc_finishes_a_norm(m, n, k, out_dtype):
    """A product over rows that were multiplied by a norm's weights but not divided by their root mean square,
    with the rows' sums of squares in parts: equal to the product over the normalised rows."""
    eps = 1e-5
    g = torch.Generator().manual_seed(m + n + k)
    stream = 5 * torch.randn(m, k, generator=g) * (1 + torch.arange(m).float()[:, None])      # rows of very different size
    norm_w = 1 + 0.2 * torch.randn(k, generator=g)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    scaled = (stream * norm_w).to(torch.bfloat16)
    parts = 3
    stride = 48
    sums = torch.zeros(parts, stride)
    cut = [0, k // 3, k // 2, k]
    for p in range(parts):
        sums[p, :m] = (stream[:, cut[p]:cut[p + 1]] ** 2).sum(1)
    out = torch.full((m, n), float("nan"), dtype=out_dtype, device=DEV)
    kernels.gemm_tc(scaled.to(DEV), w.to(DEV), out, row_sums=(sums.to(DEV), k, eps))
    torch.cuda.synchronize()
    kernels.check_device_errors()
    factor = torch.rsqrt((stream.double() ** 2).mean(1, keepdim=True) + eps)
    normed = stream.double() * factor * norm_w.double()
    close(out, normed @ w.double().T, torch.bfloat16, "product over the normalised rows")     # x was rounded to bfloat16


@pytest.mark.parametrize("m", [1, 8])
def test_gemm_tc_gated_and_heads_finish_a_norm(m):
    """The same through the gated epilogue and through the q/k/v epilogue (whose head norms are not invariant
    under the factor, because of their eps)."""
    eps, k, inner, nq, nkv, d, page, pages, theta = 1e-6, 1024, 384, 4, 2, 128, 16, 4, 1e4
    g = torch.Generator().manual_seed(m)
    stream = 0.01 * torch.randn(m, k, generator=g)                         # small rows: the factor is large
    norm_w = 1 + 0.2 * torch.randn(k, generator=g)
    scaled = (stream * norm_w).to(torch.bfloat16)
    sums = torch.zeros(2, 16)
    sums[0, :m] = (stream[:, :600] ** 2).sum(1)
    sums[1, :m] = (stream[:, 600:] ** 2).sum(1)
    factor = torch.rsqrt((stream.double() ** 2).mean(1, keepdim=True) + eps)
    normed = scaled.double() * factor                                       # the rounding that the kernel sees
    gate = (torch.randn(inner, k, generator=g) / k ** 0.5 * 2).to(torch.bfloat16)
    up = (torch.randn(inner, k, generator=g) / k ** 0.5 * 2).to(torch.bfloat16)
    mixed = torch.stack([gate.view(-1, 64, k), up.view(-1, 64, k)], dim=1).reshape(2 * inner, k).contiguous()
    act = torch.full((m, inner), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.gemm_tc(scaled.to(DEV), mixed.to(DEV), act, gated=True, row_sums=(sums.to(DEV), k, eps))
    gd, ud = normed @ gate.double().T, normed @ up.double().T
    close(act, gd / (1 + torch.exp(-gd)) * ud, torch.bfloat16, "gated")
    w = (torch.randn((nq + 2 * nkv) * d, k, generator=g) / k ** 0.5 * 0.02).to(torch.bfloat16)     # head norms feel their eps
    q_w, k_w = 1 + 0.1 * torch.randn(d, generator=g), 1 + 0.1 * torch.randn(d, generator=g)
    positions = torch.randint(0, 3000, (m,), generator=g, dtype=torch.int32)
    slots = torch.randperm(pages * page, generator=g)[:m].to(torch.int32)
    inv_freq = RotaryPosition.inverse_frequencies(d, theta)
    q_out = torch.full((m, nq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros(pages, nkv, page, d, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    kernels.gemm_tc_qkv_heads(scaled.to(DEV), w.to(DEV), q_out, kc, vc, positions.to(DEV), slots.to(DEV), q_w.to(DEV), k_w.to(DEV),
                              1e-3, inv_freq.to(DEV), nq, nkv, row_sums=(sums.to(DEV), k, eps))
    torch.cuda.synchronize()
    kernels.check_device_errors()
    qkv = (normed @ w.double().T).float()
    q, kk, v = plain_qk(qkv.to(DEV), positions.to(DEV), q_w.to(DEV), k_w.to(DEV), 1e-3, theta, nq, nkv, d)
    close(q_out.view(m, nq, d), q, torch.bfloat16, "q")
    slot = slots.long()
    close(kc.cpu()[slot // page, :, slot % page], kk, torch.bfloat16, "k in the cache")
    close(vc.cpu()[slot // page, :, slot % page], v, torch.bfloat16, "v in the cache")


def test_gemm_tc_rows_do_not_depend_on_the_batch():
    """The same row alone, among 8 and among 100 others: equal bit for bit, twice in a row (the
    counters of the ranges of K are left ready for the next launch)."""
    g = torch.Generator().manual_seed(5)
    n, k = 4096, 4096
    x = torch.randn(100, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) / 64).to(torch.bfloat16).to(DEV)
    outs = []
    for m in (1, 8, 100, 1):
        out = torch.empty((m, n), dtype=torch.float32, device=DEV)
        kernels.gemm_tc(x[:m].contiguous(), w, out)
        outs.append(out[0].clone())
    torch.cuda.synchronize()
    kernels.check_device_errors()
    for other in outs[1:]:
        assert torch.equal(outs[0], other)
    assert not kernels.gemm_tc_supported(x[:, :100].contiguous(), w[:, :100].contiguous())      # rows of 200 bytes
    assert not kernels.gemm_tc_supported(torch.zeros(129, 64, dtype=torch.bfloat16, device=DEV), w[:, :64].contiguous())


# --------------------------------------------------------------------------------- sampling
def test_argmax_takes_the_smaller_id_on_a_tie():
    logits = torch.randn(6, 1000, device=DEV)
    logits[0, 17] = logits[0, 900] = 50.0
    logits[1, 999] = 60.0
    logits[2, 0] = 60.0
    logits[3] = 0.0
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    kernels.argmax(logits, out)
    want = [17, 999, 0, 0] + [int(logits[i].argmax()) for i in (4, 5)]
    assert out.tolist() == want


@pytest.mark.parametrize("vocab", [16384, 70001, 151936])
def test_argmax_of_long_rows_shared_by_a_cluster(vocab):
    """Rows long enough to be shared by the blocks of a cluster: ties across shares, the last id,
    a share's edge."""
    logits = torch.randn(5, vocab, device=DEV)
    share = -(-vocab // (8 if vocab >= 65536 else 4))
    logits[0, 5] = logits[0, vocab - 1] = 40.0          # a tie between the first and the last share
    logits[1, vocab - 1] = 41.0
    logits[2, share - 1] = logits[2, share] = 42.0      # a tie across a share's edge
    logits[3, share] = 43.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    kernels.argmax(logits, out)
    assert out.tolist() == [5, vocab - 1, share - 1, share, int(logits[4].argmax())]


def plain_draw(logits, params: SamplingParams, index: int) -> int:
    """The kernel's draw restated: the reference's support, then the inverse CDF in id order."""
    ids, weights = P.nucleus_support(logits.double().cpu(), params.temperature, params.top_k, params.top_p)
    pairs = sorted(zip(ids, weights))
    u = uniform_from_counter(params.seed, index) * sum(w for _, w in pairs)
    run = 0.0
    for i, w in pairs:
        run += w
        if run > u:
            return i
    return pairs[-1][0]


@pytest.mark.parametrize("vocab", [3, 301, 5000])
def test_sampler_support_and_repeatability(vocab):
    sampler = Sampler(torch.device(DEV))
    g = torch.Generator().manual_seed(vocab)
    logits = (torch.randn(1, vocab, generator=g) * 2).to(DEV)
    settings = [SamplingParams(temperature=1.0, seed=42), SamplingParams(temperature=0.7, top_k=2, top_p=0.9, seed=42),
                SamplingParams(temperature=1.3, top_p=0.5, seed=7), SamplingParams(temperature=0.5, top_k=min(50, vocab), seed=9),
                SamplingParams(temperature=2.0, top_k=vocab + 5, top_p=0.999, seed=11)]
    for params in settings:
        support, _ = P.nucleus_support(logits[0].cpu(), params.temperature, params.top_k, params.top_p)
        draws = 200
        rows = logits.expand(draws, vocab).contiguous()
        got = sampler.sample(rows, [params] * draws, list(range(draws)))
        assert got == sampler.sample(rows, [params] * draws, list(range(draws)))      # same seed, same draws
        assert set(got) <= set(support), f"drew outside the support with {params}"
        want = [plain_draw(logits[0], params, i) for i in range(draws)]
        agree = sum(a == b for a, b in zip(got, want))
        assert agree >= draws - 2, f"{draws - agree} of {draws} draws differ from the plain draw with {params}"
    tiny = SamplingParams(temperature=1.0, top_k=2, top_p=0.01, seed=1)
    assert set(sampler.sample(logits.expand(20, vocab).contiguous(), [tiny] * 20, list(range(20)))) == {int(logits[0].argmax())}


def test_sampler_distribution_ties_and_bad_rows():
    sampler = Sampler(torch.device(DEV))
    logits = torch.tensor([[0.0, 2.0, 1.0, -1.0, 0.5]], device=DEV)
    params = SamplingParams(temperature=0.7, seed=3)
    draws = 4000
    got = sampler.sample(logits.expand(draws, 5).contiguous(), [params] * draws, list(range(draws)))
    probs = torch.softmax(logits[0].double().cpu() / 0.7, 0)
    counts = torch.bincount(torch.tensor(got), minlength=5).double()
    chi2 = ((counts - draws * probs) ** 2 / (draws * probs)).sum().item()
    assert chi2 < 25.0, f"chi-square {chi2:.1f} over 4 degrees of freedom"
    # all logits equal, top_k 3: the three smallest ids, as the reference's sort by (value, id) keeps them
    flat = torch.zeros(300, 40, device=DEV)
    got = sampler.sample(flat, [SamplingParams(temperature=1.0, top_k=3, seed=5)] * 300, list(range(300)))
    assert set(got) == {0, 1, 2}
    got = sampler.sample(flat, [SamplingParams(temperature=1.0, top_p=0.1, seed=5)] * 300, list(range(300)))
    assert set(got) == {0, 1, 2, 3}
    # greedy rows beside sampled rows
    mixed = sampler.sample(logits.expand(3, 5).contiguous(),
                           [SamplingParams(), SamplingParams(temperature=0.9, top_k=1), params], [0, 0, 0])
    assert mixed[0] == 1 and mixed[1] == 1
    bad = logits.clone()
    bad[0, 2] = float("nan")
    with pytest.raises(BackendError, match="nonfinite"):
        sampler.sample(bad, [params], [0])
    bad[0, 2] = float("inf")
    with pytest.raises(BackendError, match="nonfinite"):
        sampler.sample(bad, [params], [0])
