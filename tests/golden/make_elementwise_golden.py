#!/usr/bin/env python3
"""Makes tests/golden/elementwise_golden.json.

The reference's whole model cannot be built on a CPU (Rust host code over CUDA
kernels), but four of its elementwise CUDA sources are plain C once the CUDA
keywords are defined away: this script compiles them *from the reference
checkout, unchanged* with g++ behind a small shim that runs a kernel as a 1x1
launch, calls them on fixed inputs and stores inputs and outputs.  The test
`tests/test_plain.py::test_formulas_match_the_reference_sources` then holds the
plain implementation to them.  Run once by hand:

    python tests/golden/make_elementwise_golden.py /path/to/reference

Nothing of the reference is copied into this repository; only numbers are kept.
Sources used: src/kernels_cuda/rmsnorm.cuh (rmsnorm_rms_inv),
src/kernels_cuda/rope.cu (rope_kernel), src/kernels_cuda/silu_and_mul.cu
(silu_and_mul_kernel), src/kernels_cuda/elementwise.cu (add_kernel).
"""

import json
import os
import subprocess
import sys
import tempfile

import numpy as np

SHIM = r"""
#include <cmath>
#include <cstdio>
#include <cstdlib>
#define __global__
#define __device__
#define __restrict__
#define __forceinline__ inline
struct dim3_ { unsigned int x, y, z; };
static dim3_ threadIdx = {0, 0, 0}, blockIdx = {0, 0, 0}, blockDim = {1, 1, 1}, gridDim = {1, 1, 1};
struct float4 { float x, y, z, w; };
#include "rmsnorm.cuh"
#include "rope.cu"
#include "silu_and_mul.cu"
#define moe_scatter_add_kernel moe_scatter_add_kernel_unused
static inline float atomicAdd(float* p, float v) { float o = *p; *p += v; return o; }
static inline unsigned int min(unsigned int a, unsigned int b) { return a < b ? a : b; }
#include "elementwise.cu"

int main(int argc, char** argv) {
    // argv: op then numbers on stdin
    FILE* in = stdin;
    char op[32];
    if (fscanf(in, "%31s", op) != 1) return 1;
    int n;
    if (std::string(op) == "rmsnorm") {
        float eps; fscanf(in, "%d %f", &n, &eps);
        float* x = (float*)aligned_alloc(16, sizeof(float) * ((n + 3) / 4 * 4));
        for (int i = 0; i < n; ++i) fscanf(in, "%f", &x[i]);
        printf("%.9g\n", rmsnorm_rms_inv(x, (unsigned)n, eps, false));
    } else if (std::string(op) == "rope") {
        int heads, d, rd, pos; float base;
        fscanf(in, "%d %d %d %d %f", &heads, &d, &rd, &pos, &base);
        n = heads * d;
        float* x = (float*)malloc(sizeof(float) * n);
        for (int i = 0; i < n; ++i) fscanf(in, "%f", &x[i]);
        rope_kernel(x, (unsigned)pos, heads, d, rd, base);
        for (int i = 0; i < n; ++i) printf("%.9g\n", x[i]);
    } else if (std::string(op) == "silu") {
        fscanf(in, "%d", &n);
        float *g = (float*)malloc(4 * n), *u = (float*)malloc(4 * n), *y = (float*)malloc(4 * n);
        for (int i = 0; i < n; ++i) fscanf(in, "%f", &g[i]);
        for (int i = 0; i < n; ++i) fscanf(in, "%f", &u[i]);
        silu_and_mul_kernel(g, u, y, 1, n);
        for (int i = 0; i < n; ++i) printf("%.9g\n", y[i]);
    } else if (std::string(op) == "add") {
        fscanf(in, "%d", &n);
        float *a = (float*)malloc(4 * n), *b = (float*)malloc(4 * n);
        for (int i = 0; i < n; ++i) fscanf(in, "%f", &a[i]);
        for (int i = 0; i < n; ++i) fscanf(in, "%f", &b[i]);
        add_kernel(a, b, n, n);
        for (int i = 0; i < n; ++i) printf("%.9g\n", a[i]);
    }
    return 0;
}
"""


def main() -> int:
    if len(sys.argv) < 2:
        print("usage: make_elementwise_golden.py <checkout of the reference>", file=sys.stderr)
        return 2
    ref = sys.argv[1]
    kdir = os.path.join(ref, "src", "kernels_cuda")
    tmp = tempfile.mkdtemp()
    src = os.path.join(tmp, "shim.cpp")
    with open(src, "w") as f:
        f.write("#include <string>\n" + SHIM)
    exe = os.path.join(tmp, "shim")
    subprocess.run(["g++", "-O1", "-w", "-std=c++17", "-x", "c++", "-I", kdir, src, "-o", exe], check=True)

    def call(text: str):
        out = subprocess.run([exe], input=text, capture_output=True, text=True, check=True).stdout
        return [float(x) for x in out.split()]

    def f32(a):
        return [float(np.float32(v)) for v in a]

    rng = np.random.default_rng(20240607)
    gold = {}
    x = f32(rng.normal(size=100) * 1.5)
    eps = 1e-6
    (inv,) = call("rmsnorm %d %g\n%s\n" % (len(x), eps, " ".join(repr(v) for v in x)))
    gold["rmsnorm"] = {"x": x, "eps": eps, "rms_inv": inv}
    gold["rope"] = []
    for heads, d, rd, pos, base in ((2, 16, 16, 0, 1e4), (3, 32, 32, 17, 1e6), (1, 48, 32, 1000, 5e4), (2, 16, 16, 4095, 1e4)):
        t = f32(rng.normal(size=heads * d))
        y = call("rope %d %d %d %d %g\n%s\n" % (heads, d, rd, pos, base, " ".join(repr(v) for v in t)))
        # the reference computes the angle in 32-bit: its error grows with the position
        atol = 4e-6 + 3e-7 * pos
        gold["rope"].append({"heads": heads, "head_dim": d, "rotary_dim": rd, "pos": pos, "base": base,
                             "x": t, "y": y, "atol": atol})
    g, u = f32(rng.normal(size=40) * 3), f32(rng.normal(size=40))
    y = call("silu %d\n%s\n%s\n" % (len(g), " ".join(map(repr, g)), " ".join(map(repr, u))))
    gold["silu_and_mul"] = {"gate": g, "up": u, "y": y}
    a, b = f32(rng.normal(size=20)), f32(rng.normal(size=20))
    y = call("add %d\n%s\n%s\n" % (len(a), " ".join(map(repr, a)), " ".join(map(repr, b))))
    gold["add"] = {"a": a, "b": b, "y": y}
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "elementwise_golden.json")
    with open(out, "w") as f:
        json.dump(gold, f)
    print("wrote", out, os.path.getsize(out), "bytes")
    return 0


if __name__ == "__main__":
    sys.exit(main())
