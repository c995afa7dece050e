"""Makes `tests/golden/elementwise.npz`: the reference's own one-thread-per-element kernels
(crates/kernels/src/ops.cu: `add`, `rope`, `swiglu`, `split_columns`, `scatter`, `embedding`)
compiled as plain C++ for the CPU and run thread by thread on small seeded inputs.

The reference's model code is Rust over a CUDA backend and cannot be built here, and its
kernels that work a block together (`rms`, `attention`, `argmax`: shuffles, barriers) make no
sense thread by thread; the kernels that compute one element a thread do, and they fix where
the reference rounds to bfloat16.  `tests/test_plain.py` compares the plain implementation's
bfloat16 mode with these outputs bit for bit.

    python tests/golden/make_golden.py --reference PATH_TO_mini-rsglang [--cuda /usr/local/cuda]

Needs g++ and the CUDA headers (`cuda_bf16.h` has host versions of the conversions).  The
file it writes is committed, so the tests need neither."""
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
#include <cstring>
#include <vector>
#include <algorithm>
#include <cuda_bf16.h>
struct Index { unsigned x, y, z; };
static Index threadIdx, blockIdx, blockDim, gridDim;
#undef __global__
#undef __device__
#undef __shared__
#define __global__
#define __device__
#define __shared__ static
static inline void __syncthreads() {}
static inline float __shfl_down_sync(unsigned, float, int) { return 0.0f; }     // only in kernels that are not run here
static inline float rsqrtf(float x) { return 1.0f / sqrtf(x); }
static inline float __int_as_float(unsigned bits) { float v; memcpy(&v, &bits, 4); return v; }
using std::max;
using std::min;
#include "OPS_CU"

// Runs a kernel of `threads` one-element threads in blocks of 256.
template <typename F> static void run(int threads, F kernel) {
    blockDim = {256, 1, 1};
    for (int i = 0; i < threads; ++i) {
        blockIdx = {(unsigned)(i / 256), 0, 0};
        threadIdx = {(unsigned)(i % 256), 0, 0};
        kernel();
    }
}
static std::vector<uint16_t> read16(const char* path, size_t n) {
    std::vector<uint16_t> v(n);
    FILE* f = fopen(path, "rb");
    if (!f || fread(v.data(), 2, n, f) != n) { fprintf(stderr, "cannot read %s\n", path); exit(1); }
    fclose(f);
    return v;
}
static std::vector<uint32_t> read32(const char* path, size_t n) {
    std::vector<uint32_t> v(n);
    FILE* f = fopen(path, "rb");
    if (!f || fread(v.data(), 4, n, f) != n) { fprintf(stderr, "cannot read %s\n", path); exit(1); }
    fclose(f);
    return v;
}
static void write16(const char* path, const std::vector<uint16_t>& v) {
    FILE* f = fopen(path, "wb");
    fwrite(v.data(), 2, v.size(), f);
    fclose(f);
}
int main(int argc, char** argv) {
    const int n = atoi(argv[1]), heads = atoi(argv[2]), d = atoi(argv[3]), width = atoi(argv[4]), vocab = atoi(argv[5]);
    // add
    auto x = read16("x.bin", (size_t)n * width), y = read16("y.bin", (size_t)n * width);
    std::vector<uint16_t> z((size_t)n * width);
    run(n * width, [&] { add((const bf16*)x.data(), (const bf16*)y.data(), (bf16*)z.data(), n * width); });
    write16("add.bin", z);
    // swiglu
    run(n * width, [&] { swiglu((const bf16*)x.data(), (const bf16*)y.data(), (bf16*)z.data(), n * width); });
    write16("swiglu.bin", z);
    // rope, in place on a copy of q [n, heads, d]
    auto q = read16("q.bin", (size_t)n * heads * d);
    auto pos = read32("pos.bin", n);
    auto freq = read32("freq.bin", d / 2);
    run(n * heads * (d / 2), [&] { rope((bf16*)q.data(), pos.data(), (const float*)freq.data(), n, heads, d); });
    write16("rope.bin", q);
    // split_columns: columns [start, start + part) of x [n, width]
    const int start = width / 4, part = width / 2;
    std::vector<uint16_t> cols((size_t)n * part);
    run(n * part, [&] { split_columns((const bf16*)x.data(), (bf16*)cols.data(), n, width, start, part); });
    write16("split.bin", cols);
    // scatter of x and y rows into caches of 2 n rows at `slots`
    auto slots = read32("slots.bin", n);
    std::vector<uint16_t> kc((size_t)2 * n * width, 0), vc((size_t)2 * n * width, 0);
    run(n * width, [&] { scatter((const bf16*)x.data(), (const bf16*)y.data(), slots.data(), (bf16*)kc.data(), (bf16*)vc.data(), n, width); });
    write16("kcache.bin", kc);
    write16("vcache.bin", vc);
    // embedding
    auto table = read16("table.bin", (size_t)vocab * width);
    auto ids = read32("ids.bin", n);
    run(n * width, [&] { embedding((const bf16*)table.data(), ids.data(), (bf16*)z.data(), n, width); });
    write16("embedding.bin", z);
    return 0;
}
"""


def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (round to nearest even), as uint16."""
    u = a.astype(np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of mirthfulLee/mini-rsglang")
    ap.add_argument("--cuda", default="/usr/local/cuda")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "elementwise.npz"))
    args = ap.parse_args()
    ops = os.path.join(args.reference, "crates", "kernels", "src", "ops.cu")
    n, heads, d, width, vocab, theta = 7, 3, 48, 40, 29, 50000.0
    rng = np.random.default_rng(20240607)
    x = to_bf16_bits(rng.standard_normal((n, width)) * 3)
    y = to_bf16_bits(rng.standard_normal((n, width)) * 3)
    q = to_bf16_bits(rng.standard_normal((n, heads, d)))
    pos = np.array([0, 1, 2, 17, 300, 4095, 40000], dtype=np.uint32)
    # the reference's frequency table: the power in float64, narrowed, the reciprocal in float32 (crates/kernels/src/lib.rs:612-614)
    freq = np.array([np.float32(1.0) / np.float32(float(theta) ** (2.0 * j / d)) for j in range(d // 2)], dtype=np.float32)
    slots = rng.permutation(2 * n)[:n].astype(np.uint32)
    table = to_bf16_bits(rng.standard_normal((vocab, width)))
    ids = rng.integers(0, vocab, n).astype(np.uint32)
    with tempfile.TemporaryDirectory() as tmp:
        for name, arr in (("x", x), ("y", y), ("q", q), ("pos", pos), ("freq", freq), ("slots", slots), ("table", table), ("ids", ids)):
            arr.tofile(os.path.join(tmp, name + ".bin"))
        with open(os.path.join(tmp, "harness.cc"), "w") as f:
            f.write(HARNESS.replace("OPS_CU", ops))
        subprocess.run(["g++", "-O1", "-ffp-contract=off", "-w", "-I", os.path.join(args.cuda, "include"), "-o", "harness", "harness.cc"],
                       cwd=tmp, check=True)
        subprocess.run(["./harness", str(n), str(heads), str(d), str(width), str(vocab)], cwd=tmp, check=True)
        out = {name: np.fromfile(os.path.join(tmp, name + ".bin"), dtype=np.uint16)
               for name in ("add", "swiglu", "rope", "split", "kcache", "vcache", "embedding")}
    np.savez_compressed(args.out, x=x, y=y, q=q, pos=pos, freq=freq, slots=slots, table=table, ids=ids, theta=np.float64(theta),
                        add=out["add"].reshape(n, width), swiglu=out["swiglu"].reshape(n, width),
                        rope=out["rope"].reshape(n, heads, d), split=out["split"].reshape(n, width // 2),
                        kcache=out["kcache"].reshape(2 * n, width), vcache=out["vcache"].reshape(2 * n, width),
                        embedding=out["embedding"].reshape(n, width))
    print(args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    main()
