"""Makes `tests/golden/model.npz`: the reference's kernels that work a block together (`rms`, `attention`,
`argmax` of crates/kernels/src/ops.cu) and a whole tiny Qwen3 forward pass made of the reference's own kernels,
all compiled as plain C++ and run on the CPU.

The reference's model code is Rust over a CUDA backend and cannot be built here (no Rust toolchain, no GPU);
its one CUDA source can.  A kernel's block runs as one fiber per CUDA thread: `__syncthreads()` and the warp
shuffles hand over to the next fiber, so the threads of a block advance from barrier to barrier together, which
is what the kernels assume.  The forward pass calls those kernels in the order of `forward_hidden_observed` and
`project` (crates/models/src/qwen3.rs:160-236: embedding; per layer rms, q/k/v projection, split, per-head rms of q
and k, rope, scatter into the paged cache, attention, o projection, add, rms, gate/up projection, split, swiglu,
down projection, add; the last rms; the head with float32 output), with the projections, which the reference leaves
to a library, as plain sums in float64 rounded once.  The order of the calls is this script's reading of that Rust
source; every kernel that is called is the reference's own text.

    python tests/golden/make_model_golden.py --reference PATH_TO_mini-rsglang [--cuda /usr/local/cuda]

Needs g++ and the CUDA headers.  The file it writes is committed, so the tests need neither;
`tests/test_plain.py` compares the plain implementation with it."""
from __future__ import annotations

import argparse
import os
import subprocess
import tempfile

import numpy as np

HARNESS = r"""
#include <cmath>
#include <cstdio>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <vector>
#include <algorithm>
#include <ucontext.h>
#include <cuda_bf16.h>
struct Index { unsigned x, y, z; };
static Index threadIdx, blockIdx, blockDim, gridDim;
#undef __global__
#undef __device__
#undef __shared__
#define __global__
#define __device__
#define __shared__ static

// ---- a block of CUDA threads as fibers: every barrier hands over to the next thread --------------------------
static ucontext_t scheduler_context;
static std::vector<ucontext_t> fibers;
static std::vector<char> finished;
static int current = 0;
static std::function<void()>* body = nullptr;
static float exchange[1024];
static void barrier() { swapcontext(&fibers[current], &scheduler_context); }
static inline void __syncthreads() { barrier(); }
// every thread of the block calls the shuffle at the same place (true of the kernels that are run here)
static inline float __shfl_down_sync(unsigned, float x, int offset) {
    const int me = current;
    exchange[me] = x;
    barrier();
    const int lane = me % 32;
    const float got = lane + offset < 32 ? exchange[me + offset] : x;
    barrier();
    return got;
}
static inline float rsqrtf(float x) { return 1.0f / sqrtf(x); }
static inline float __int_as_float(unsigned bits) { float v; memcpy(&v, &bits, 4); return v; }
using std::max;
using std::min;
#include "OPS_CU"

static void fiber_entry() {
    (*body)();
    finished[current] = 1;
    swapcontext(&fibers[current], &scheduler_context);
}
// Runs kernel() for every thread of a grid_x * grid_y grid of blocks of `threads` threads.
static void launch(unsigned grid_x, unsigned grid_y, unsigned threads, std::function<void()> kernel) {
    static std::vector<std::vector<char>> stacks;
    const size_t stack_bytes = 256 * 1024;
    if (stacks.size() < threads) stacks.resize(threads, std::vector<char>(stack_bytes));
    body = &kernel;
    blockDim = {threads, 1, 1};
    gridDim = {grid_x, grid_y, 1};
    for (unsigned by = 0; by < grid_y; ++by)
        for (unsigned bx = 0; bx < grid_x; ++bx) {
            blockIdx = {bx, by, 0};
            fibers.assign(threads, ucontext_t());
            finished.assign(threads, 0);
            for (unsigned t = 0; t < threads; ++t) {
                getcontext(&fibers[t]);
                fibers[t].uc_stack.ss_sp = stacks[t].data();
                fibers[t].uc_stack.ss_size = stack_bytes;
                fibers[t].uc_link = &scheduler_context;
                makecontext(&fibers[t], fiber_entry, 0);
            }
            bool any = true;
            while (any) {                  // one round = every thread from one barrier to the next
                any = false;
                for (unsigned t = 0; t < threads; ++t) {
                    if (finished[t]) continue;
                    current = (int)t;
                    threadIdx = {t, 0, 0};
                    swapcontext(&scheduler_context, &fibers[t]);
                    if (!finished[t]) any = true;
                }
            }
        }
}
static void launch_flat(size_t elements, std::function<void()> kernel) {      // one element a thread, blocks of 256
    launch((unsigned)((elements + 255) / 256), 1, 256, kernel);
}

template <typename T> static std::vector<T> read_file(const char* path, size_t n) {
    std::vector<T> v(n);
    FILE* f = fopen(path, "rb");
    if (!f || fread(v.data(), sizeof(T), n, f) != n) { fprintf(stderr, "cannot read %s\n", path); exit(1); }
    fclose(f);
    return v;
}
template <typename T> static void write_file(const char* path, const std::vector<T>& v) {
    FILE* f = fopen(path, "wb");
    fwrite(v.data(), sizeof(T), v.size(), f);
    fclose(f);
}
typedef std::vector<uint16_t> Bits;       // bfloat16 bit patterns
static float as_float(uint16_t h) { unsigned u = (unsigned)h << 16; float v; memcpy(&v, &u, 4); return v; }
static uint16_t round_bf16(float x) { __nv_bfloat16 h = __float2bfloat16_rn(x); uint16_t u; memcpy(&u, &h, 2); return u; }
// y[M, N] = x[M, K] . w[N, K]^T: the sum in float64, rounded to float32 and then (unless `keep32`) to bfloat16
static void project(const Bits& x, const Bits& w, int M, int N, int K, Bits* out16, std::vector<float>* out32) {
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            double sum = 0;
            for (int k = 0; k < K; ++k) sum += (double)as_float(x[(size_t)m * K + k]) * (double)as_float(w[(size_t)n * K + k]);
            if (out16) (*out16)[(size_t)m * N + n] = round_bf16((float)sum);
            if (out32) (*out32)[(size_t)m * N + n] = (float)sum;
        }
}
static Bits rms_rows(const Bits& x, const Bits& w, int rows, int d, float eps) {
    Bits out(x.size());
    launch(rows, 1, 256, [&] { rms((const bf16*)x.data(), (const bf16*)w.data(), (bf16*)out.data(), d, eps); });
    return out;
}
static Bits columns(const Bits& x, int n, int full, int start, int width) {
    Bits out((size_t)n * width);
    launch_flat((size_t)n * width, [&] { split_columns((const bf16*)x.data(), (bf16*)out.data(), n, full, start, width); });
    return out;
}
static Bits sum_of(const Bits& x, const Bits& y) {
    Bits out(x.size());
    launch_flat(x.size(), [&] { add((const bf16*)x.data(), (const bf16*)y.data(), (bf16*)out.data(), (int)x.size()); });
    return out;
}

int main(int argc, char** argv) {
    // ---------------------------------------------------------------- the kernels alone
    {
        const int rows = atoi(argv[1]), d = atoi(argv[2]);
        auto x = read_file<uint16_t>("rms_x.bin", (size_t)rows * d), w = read_file<uint16_t>("rms_w.bin", d);
        write_file("rms_out.bin", rms_rows(x, w, rows, d, 1e-5f));
    }
    {
        // a mixed batch over scrambled pages: some tokens that continue a request, and a fresh prompt
        const int tokens = atoi(argv[3]), qheads = atoi(argv[4]), kvheads = atoi(argv[5]), d = atoi(argv[6]), page = atoi(argv[7]),
                  pages = atoi(argv[8]), width = atoi(argv[9]), window = atoi(argv[10]);
        auto q = read_file<uint16_t>("att_q.bin", (size_t)tokens * qheads * d);
        auto kc = read_file<uint16_t>("att_kc.bin", (size_t)pages * page * kvheads * d), vc = read_file<uint16_t>("att_vc.bin", (size_t)pages * page * kvheads * d);
        auto pos = read_file<uint32_t>("att_pos.bin", tokens), seq = read_file<uint32_t>("att_seq.bin", tokens);
        auto table = read_file<uint32_t>("att_table.bin", (size_t)2 * width);
        Bits out((size_t)tokens * qheads * d);
        const float scale_q = (float)pow((double)d, -0.25);
        launch(tokens, qheads, 128, [&] { attention((const bf16*)q.data(), (const bf16*)kc.data(), (const bf16*)vc.data(), pos.data(), seq.data(),
                                                    table.data(), (bf16*)out.data(), qheads, kvheads, d, page, width, scale_q, nullptr, 0, 0); });
        write_file("att_out.bin", out);
        launch(tokens, qheads, 128, [&] { attention((const bf16*)q.data(), (const bf16*)kc.data(), (const bf16*)vc.data(), pos.data(), seq.data(),
                                                    table.data(), (bf16*)out.data(), qheads, kvheads, d, page, width, scale_q, nullptr, window, 0); });
        write_file("att_window_out.bin", out);
    }
    {
        const int rows = atoi(argv[11]), vocab = atoi(argv[12]);
        auto logits = read_file<float>("argmax_x.bin", (size_t)rows * vocab);
        std::vector<uint32_t> picked(rows);
        launch(rows, 1, 256, [&] { argmax(logits.data(), picked.data(), vocab); });
        write_file("argmax_out.bin", picked);
    }
    // ---------------------------------------------------------------- a whole forward pass (crates/models/src/qwen3.rs:160-236)
    const int L = atoi(argv[13]), H = atoi(argv[14]), nq = atoi(argv[15]), nkv = atoi(argv[16]), d = atoi(argv[17]), I = atoi(argv[18]),
              V = atoi(argv[19]), T = atoi(argv[20]), S = atoi(argv[21]);
    const float eps = (float)atof(argv[22]);
    const int pages = (T + S - 1) / S, width = pages;
    auto ids = read_file<uint32_t>("m_ids.bin", T);
    auto freq = read_file<float>("m_freq.bin", d / 2);
    auto embed = read_file<uint16_t>("m_embed.bin", (size_t)V * H), head = read_file<uint16_t>("m_head.bin", (size_t)V * H);
    auto final_norm = read_file<uint16_t>("m_norm.bin", H);
    std::vector<uint32_t> pos(T), seq(T, 0), slots(T), table(width);
    for (int p = 0; p < pages; ++p) table[p] = (uint32_t)(pages - 1 - p);          // pages in reverse order
    for (int t = 0; t < T; ++t) pos[t] = t, slots[t] = table[t / S] * S + t % S;
    Bits x((size_t)T * H);
    launch_flat((size_t)T * H, [&] { embedding((const bf16*)embed.data(), ids.data(), (bf16*)x.data(), T, H); });
    const int qw = nq * d, kw = nkv * d;
    const float scale_q = (float)pow((double)d, -0.25);
    for (int layer = 0; layer < L; ++layer) {
        char name[64];
        auto weight = [&](const char* leaf, size_t n) { snprintf(name, sizeof name, "m_l%d_%s.bin", layer, leaf); return read_file<uint16_t>(name, n); };
        auto in_norm = weight("in_norm", H), post_norm = weight("post_norm", H), q_norm = weight("q_norm", d), k_norm = weight("k_norm", d);
        auto w_qkv = weight("qkv", (size_t)(qw + 2 * kw) * H), w_o = weight("o", (size_t)H * qw);
        auto w_gu = weight("gate_up", (size_t)2 * I * H), w_down = weight("down", (size_t)H * I);
        Bits n1 = rms_rows(x, in_norm, T, H, eps);
        Bits qkv((size_t)T * (qw + 2 * kw));
        project(n1, w_qkv, T, qw + 2 * kw, H, &qkv, nullptr);
        Bits q = columns(qkv, T, qw + 2 * kw, 0, qw), k = columns(qkv, T, qw + 2 * kw, qw, kw), v = columns(qkv, T, qw + 2 * kw, qw + kw, kw);
        q = rms_rows(q, q_norm, T * nq, d, eps);
        k = rms_rows(k, k_norm, T * nkv, d, eps);
        launch_flat((size_t)T * nq * (d / 2), [&] { rope((bf16*)q.data(), pos.data(), freq.data(), T, nq, d); });
        launch_flat((size_t)T * nkv * (d / 2), [&] { rope((bf16*)k.data(), pos.data(), freq.data(), T, nkv, d); });
        Bits kc((size_t)pages * S * kw, 0), vc((size_t)pages * S * kw, 0);
        launch_flat((size_t)T * kw, [&] { scatter((const bf16*)k.data(), (const bf16*)v.data(), slots.data(), (bf16*)kc.data(), (bf16*)vc.data(), T, kw); });
        Bits att((size_t)T * qw);
        launch(T, nq, 128, [&] { attention((const bf16*)q.data(), (const bf16*)kc.data(), (const bf16*)vc.data(), pos.data(), seq.data(), table.data(),
                                           (bf16*)att.data(), nq, nkv, d, S, width, scale_q, nullptr, 0, 0); });
        Bits projected((size_t)T * H);
        project(att, w_o, T, H, qw, &projected, nullptr);
        Bits residual = sum_of(x, projected);
        Bits n2 = rms_rows(residual, post_norm, T, H, eps);
        Bits merged((size_t)T * 2 * I);
        project(n2, w_gu, T, 2 * I, H, &merged, nullptr);
        Bits gate = columns(merged, T, 2 * I, 0, I), up = columns(merged, T, 2 * I, I, I), activated((size_t)T * I);
        launch_flat((size_t)T * I, [&] { swiglu((const bf16*)gate.data(), (const bf16*)up.data(), (bf16*)activated.data(), T * I); });
        Bits down((size_t)T * H);
        project(activated, w_down, T, H, I, &down, nullptr);
        x = sum_of(residual, down);
        if (layer == 0) {
            write_file("m_l0_attn.bin", att);
            write_file("m_l0_output.bin", x);
        }
    }
    Bits last = rms_rows(x, final_norm, T, H, eps);
    std::vector<float> logits((size_t)T * V);
    project(last, head, T, V, H, nullptr, &logits);
    write_file("m_final_norm.bin", last);
    write_file("m_logits.bin", logits);
    return 0;
}
"""


def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (round to nearest even), as uint16."""
    u = a.astype(np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def frequencies(d: int, theta: float) -> np.ndarray:
    """The reference's table: the power in float64, narrowed, the reciprocal in float32 (crates/kernels/src/lib.rs:612-614)."""
    return np.array([np.float32(1.0) / np.float32(float(theta) ** (2.0 * j / d)) for j in range(d // 2)], dtype=np.float32)


MODEL = dict(layers=2, hidden=48, q_heads=6, kv_heads=2, head_dim=16, inner=80, vocab=61, tokens=21, page=4, eps=1e-5, theta=50000.0)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of mirthfulLee/mini-rsglang")
    ap.add_argument("--cuda", default="/usr/local/cuda")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "model.npz"))
    args = ap.parse_args()
    ops = os.path.join(args.reference, "crates", "kernels", "src", "ops.cu")
    rng = np.random.default_rng(20240612)
    files, kept = {}, {}

    # rms: rows of a width that is no multiple of 32
    rows, d = 5, 133
    files["rms_x"] = to_bf16_bits(rng.standard_normal((rows, d)) * 2)
    files["rms_w"] = to_bf16_bits(1 + 0.1 * rng.standard_normal(d))
    # attention: 5 tokens that continue a request at position 17 over pages [2, 5], beside a fresh prompt of 37 tokens over
    # pages [0, 8, 3] (the reference's own fixture, crates/kernels/examples/verify_ops.rs:29-47); 6 query heads on 2
    a = dict(tokens=42, q_heads=6, kv_heads=2, head_dim=48, page=16, pages=9, width=3, window=7)
    files["att_q"] = to_bf16_bits(rng.standard_normal((a["tokens"], a["q_heads"], a["head_dim"])))
    files["att_kc"] = to_bf16_bits(rng.standard_normal((a["pages"], a["page"], a["kv_heads"], a["head_dim"])))
    files["att_vc"] = to_bf16_bits(rng.standard_normal((a["pages"], a["page"], a["kv_heads"], a["head_dim"])))
    files["att_pos"] = np.array(list(range(17, 22)) + list(range(37)), dtype=np.uint32)
    files["att_seq"] = np.array([0] * 5 + [1] * 37, dtype=np.uint32)
    files["att_table"] = np.array([[2, 5, 0], [0, 8, 3]], dtype=np.uint32)
    # argmax: ties, and the largest value late in a row longer than the block
    logits = rng.standard_normal((3, 301)).astype(np.float32)
    logits[0, [17, 200]] = 9.0
    logits[1, 300] = 9.0
    files["argmax_x"] = logits
    # the model
    m = MODEL
    qw, kw = m["q_heads"] * m["head_dim"], m["kv_heads"] * m["head_dim"]

    def matrix(n, k):
        return to_bf16_bits(rng.standard_normal((n, k)) * 0.08)

    def scale(n):
        return to_bf16_bits(1 + 0.1 * rng.standard_normal(n))

    files["m_ids"] = rng.integers(0, m["vocab"], m["tokens"]).astype(np.uint32)
    files["m_freq"] = frequencies(m["head_dim"], m["theta"])
    files["m_embed"], files["m_head"], files["m_norm"] = matrix(m["vocab"], m["hidden"]), matrix(m["vocab"], m["hidden"]), scale(m["hidden"])
    for layer in range(m["layers"]):
        q, k, v = matrix(qw, m["hidden"]), matrix(kw, m["hidden"]), matrix(kw, m["hidden"])
        gate, up = matrix(m["inner"], m["hidden"]), matrix(m["inner"], m["hidden"])
        kept[f"model.layers.{layer}.self_attn.q_proj.weight"], kept[f"model.layers.{layer}.self_attn.k_proj.weight"] = q, k
        kept[f"model.layers.{layer}.self_attn.v_proj.weight"] = v
        kept[f"model.layers.{layer}.mlp.gate_proj.weight"], kept[f"model.layers.{layer}.mlp.up_proj.weight"] = gate, up
        files[f"m_l{layer}_qkv"] = np.concatenate([q, k, v])             # rows concatenated at load (qwen3.rs:73-86)
        files[f"m_l{layer}_gate_up"] = np.concatenate([gate, up])        # (qwen3.rs:255-261)
        for leaf, name, value in (("o", "self_attn.o_proj", matrix(m["hidden"], qw)), ("down", "mlp.down_proj", matrix(m["hidden"], m["inner"])),
                                  ("in_norm", "input_layernorm", scale(m["hidden"])), ("post_norm", "post_attention_layernorm", scale(m["hidden"])),
                                  ("q_norm", "self_attn.q_norm", scale(m["head_dim"])), ("k_norm", "self_attn.k_norm", scale(m["head_dim"]))):
            files[f"m_l{layer}_{leaf}"] = kept[f"model.layers.{layer}.{name}.weight"] = value
    kept["model.embed_tokens.weight"], kept["lm_head.weight"], kept["model.norm.weight"] = files["m_embed"], files["m_head"], files["m_norm"]

    with tempfile.TemporaryDirectory() as tmp:
        for name, arr in files.items():
            arr.tofile(os.path.join(tmp, name + ".bin"))
        with open(os.path.join(tmp, "harness.cc"), "w") as f:
            f.write(HARNESS.replace("OPS_CU", ops))
        subprocess.run(["g++", "-O1", "-ffp-contract=off", "-w", "-I", os.path.join(args.cuda, "include"), "-o", "harness", "harness.cc"],
                       cwd=tmp, check=True)
        argv = [rows, d, a["tokens"], a["q_heads"], a["kv_heads"], a["head_dim"], a["page"], a["pages"], a["width"], a["window"], 3, 301,
                m["layers"], m["hidden"], m["q_heads"], m["kv_heads"], m["head_dim"], m["inner"], m["vocab"], m["tokens"], m["page"], m["eps"]]
        subprocess.run(["./harness"] + [str(v) for v in argv], cwd=tmp, check=True)

        def out(name, dtype, shape):
            return np.fromfile(os.path.join(tmp, name + ".bin"), dtype=dtype).reshape(shape)

        T, H, V = m["tokens"], m["hidden"], m["vocab"]
        results = dict(
            rms_out=out("rms_out", np.uint16, (rows, d)),
            att_out=out("att_out", np.uint16, (a["tokens"], a["q_heads"] * a["head_dim"])),
            att_window_out=out("att_window_out", np.uint16, (a["tokens"], a["q_heads"] * a["head_dim"])),
            argmax_out=out("argmax_out", np.uint32, (3,)),
            m_l0_attn=out("m_l0_attn", np.uint16, (T, qw)), m_l0_output=out("m_l0_output", np.uint16, (T, H)),
            m_final_norm=out("m_final_norm", np.uint16, (T, H)), m_logits=out("m_logits", np.float32, (T, V)))
    inputs = {k: v for k, v in files.items() if not k.startswith("m_l") and k not in ("m_embed", "m_head", "m_norm")}
    weights = {"w:" + k: v for k, v in kept.items()}
    np.savez_compressed(args.out, **inputs, **weights, **results, att_shape=np.array([a[k] for k in ("tokens", "q_heads", "kv_heads", "head_dim", "page", "pages", "width", "window")]),
                        model_shape=np.array([m[k] for k in ("layers", "hidden", "q_heads", "kv_heads", "head_dim", "inner", "vocab", "tokens", "page")]),
                        model_eps=np.float64(m["eps"]), model_theta=np.float64(m["theta"]))
    print(args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    main()
