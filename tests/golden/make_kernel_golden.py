"""Outputs of the reference's own plain CUDA kernels on small cases, made once
on a GPU and committed as numbers (`kernel_golden.npz`), so that the plain
implementation under tests/ is held to the reference's code and not only to a
reading of it.

The kernels are compiled unchanged from a checkout of the reference, which this
script takes as its argument; nothing of the reference is copied into this
repository: the harness written here holds `#include` lines that name the
checkout's files, and launch code of its own.  Covered:

  src/kernels_cuda/attention.cu          attention_kernel (one query row)
  src/kernels_cuda/attention_prefill.cu  attention_prefill_kernel (rows, start_pos, window)
  src/kernels_cuda/attention_online.cu   attention_online_kernel (+ combine, key splits)
  src/kernels_cuda/gemv.cu               gemv_kernel (y = x W^T)
  src/kernels_cuda/rmsnorm.cu            rmsnorm_kernel
  src/kernels_cuda/decode_ops.cu         add_rmsnorm_kernel, rmsnorm_pair_kernel
  src/kernels_cuda/rope.cu               rope_batch_kernel

Two steps, because the machine that has the checkout and nvcc need not be the
one with the GPU:

  python tests/golden/make_kernel_golden.py build <reference checkout> <library.so>
  python tests/golden/make_kernel_golden.py run <library.so> tests/golden/kernel_golden.npz

`build` needs nvcc only (it cross-compiles for sm_100a); `run` needs a GPU and
torch (for device memory only).  Inputs are drawn from fixed seeds by
`golden_inputs` below, which the tests import to rebuild them; the file stores
outputs only.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
import sys
import tempfile

import numpy as np

# (nq, nkv, d): head counts and sizes of the attention cases (powers of two: the
# reference's plain kernels run one thread per element of a head)
HEADS = {"a": (4, 2, 16), "b": (6, 1, 32), "c": (32, 8, 128)}
# name -> (heads, rows, start_pos, window)
PREFILL_CASES = {
    "a_r129_s0_w0": ("a", 129, 0, 0),
    "a_r17_s100_w37": ("a", 17, 100, 37),
    "b_r17_s100_w0": ("b", 17, 100, 0),
    "b_r129_s0_w37": ("b", 129, 0, 37),
    "c_r1_s100_w0": ("c", 1, 100, 0),
    "c_r17_s0_w0": ("c", 17, 0, 0),
}
# the online kernel also with its keys split over blocks (no window: see the note in run())
ONLINE_SPLITS = {"b_r17_s100_w0": 3, "c_r1_s100_w0": 2}
# rows of a case that are stored (all when it has few)
KEEP_ROWS = (0, 1, 15, 16, 63, 64, 65, 128)


def kept_rows(rows: int, heads: str = "a"):
    if heads == "c":  # the wide case: first and last row only
        return sorted({0, rows - 1})
    return list(range(rows)) if rows <= 17 else [r for r in KEEP_ROWS if r < rows]


def kept_heads(heads: str):
    """Query heads of a case that are stored: every fifth of the wide case's 32
    (they fall on seven of its eight key/value heads), all of the others'."""
    nq = HEADS[heads][0]
    return list(range(0, nq, 5)) if heads == "c" else list(range(nq))


def golden_inputs(case: str):
    """The inputs of a case, from its name alone (float32 arrays)."""
    rng = np.random.default_rng(abs(hash_name(case)))
    f = lambda *shape: rng.standard_normal(shape).astype(np.float32)
    if case in PREFILL_CASES:
        heads, rows, start, _ = PREFILL_CASES[case]
        nq, nkv, d = HEADS[heads]
        return {"q": f(rows, nq, d) * 1.5, "k": f(start + rows, nkv, d), "v": f(start + rows, nkv, d)}
    if case == "gemv":
        return {"x": f(3, 96), "w": f(1000, 96) * 0.1}
    if case == "rmsnorm":
        return {"x": f(3, 96) * 2, "w": (1 + 0.1 * f(96)), "b": f(3, 96)}
    if case == "pair":
        return {"x1": f(6, 32) * 2, "w1": (1 + 0.1 * f(32)), "x2": f(2, 32) * 2, "w2": (1 + 0.1 * f(32))}
    if case == "rope":
        return {"t": f(17, 6, 32)}
    raise KeyError(case)


def hash_name(name: str) -> int:
    h = 1469598103934665603
    for ch in name.encode():
        h = ((h ^ ch) * 1099511628211) % (1 << 61)
    return h


# ----------------------------------------------------------------- the harness
# One translation unit per reference file (their headers have no include guards
# in common), each with a host launcher of this script's own.
HARNESS = {
    "attention.cu": r'''
extern "C" int gold_attention(const float* q, const float* k, const float* v, float* out, unsigned nq,
                              unsigned nkv, unsigned d, unsigned seq_len, float scale) {
    attention_kernel<<<nq, d, seq_len * sizeof(float)>>>(q, k, v, out, nq, nkv, d, seq_len, scale);
    return (int)cudaDeviceSynchronize();
}''',
    "attention_prefill.cu": r'''
extern "C" int gold_attention_prefill(const float* q, const float* k, const float* v, float* out, unsigned nq,
                                      unsigned nkv, unsigned d, unsigned start_pos, unsigned m,
                                      unsigned window, float scale) {
    attention_prefill_kernel<<<dim3(nq, m), d, (start_pos + m) * sizeof(float)>>>(
        q, k, v, out, nq, nkv, d, start_pos, m, window, scale);
    return (int)cudaDeviceSynchronize();
}''',
    "attention_online.cu": r'''
extern "C" int gold_attention_online(const float* q, const float* k, const float* v, float* out,
                                     float* partial, unsigned nq, unsigned nkv, unsigned d,
                                     unsigned start_pos, unsigned m, unsigned window, unsigned splits,
                                     float scale) {
    AttnParams p;
    p.k_pos_stride = p.v_pos_stride = (unsigned long long)nkv * d;
    p.k_head_stride = p.v_head_stride = d;
    p.num_q_heads = nq;
    p.group_size = nq / nkv;
    p.qk_dim = p.v_dim = d;
    p.start_pos = start_pos;
    p.num_splits = splits;
    p.split_len = (start_pos + m + splits - 1) / splits;
    p.window = window;
    p.scale = scale;
    const size_t smem = (d + ATTN_WARPS * (d + 2)) * sizeof(float);
    attention_online_kernel<<<dim3(m, nq, splits), ATTN_WARPS * 32, smem>>>(q, k, v, splits == 1 ? out : partial, p);
    if (splits > 1) attention_online_combine_kernel<<<dim3(m, nq), 128>>>(partial, out, nq, d, splits);
    return (int)cudaDeviceSynchronize();
}''',
    "gemv.cu": r'''
extern "C" int gold_gemv(const float* x, const float* w, float* y, unsigned in_features, unsigned out_features) {
    gemv_kernel<<<(out_features + 7) / 8, 256>>>(x, w, y, in_features, out_features);
    return (int)cudaDeviceSynchronize();
}''',
    "rmsnorm.cu": r'''
extern "C" int gold_rmsnorm(const float* x, const float* w, float* out, unsigned rows, unsigned hidden, float eps) {
    rmsnorm_kernel<<<rows, 128, hidden * sizeof(float)>>>(x, w, out, rows, hidden, eps);
    return (int)cudaDeviceSynchronize();
}''',
    "decode_ops.cu": r'''
extern "C" int gold_add_rmsnorm(float* a, const float* b, const float* w, float* out, unsigned hidden, float eps) {
    add_rmsnorm_kernel<<<1, 128, hidden * sizeof(float)>>>(a, b, w, out, hidden, eps);
    return (int)cudaDeviceSynchronize();
}
extern "C" int gold_rmsnorm_pair(const float* x1, const float* w1, float* o1, unsigned rows1, const float* x2,
                                 const float* w2, float* o2, unsigned rows2, unsigned hidden, float eps) {
    rmsnorm_pair_kernel<<<rows1 + rows2, 64, hidden * sizeof(float)>>>(x1, w1, o1, rows1, x2, w2, o2, hidden, eps);
    return (int)cudaDeviceSynchronize();
}''',
    "rope.cu": r'''
extern "C" int gold_rope_batch(float* t, unsigned start_pos, unsigned heads, unsigned d, unsigned rotary_dim,
                               unsigned m, float base) {
    rope_batch_kernel<<<8, 128>>>(t, start_pos, heads, d, rotary_dim, m, base);
    return (int)cudaDeviceSynchronize();
}''',
}


def build(reference: str, lib_path: str) -> None:
    kdir = os.path.join(os.path.abspath(reference), "src", "kernels_cuda")
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    arch = ["-gencode", "arch=compute_100a,code=sm_100a"]
    with tempfile.TemporaryDirectory() as tmp:
        objs = []
        for name, launcher in HARNESS.items():
            src = os.path.join(tmp, "harness_" + name)
            with open(src, "w") as f:
                f.write(f'#include "{os.path.join(kdir, name)}"\n#include <cuda_runtime.h>\n{launcher}\n')
            obj = src[:-3] + ".o"
            subprocess.run([nvcc, *arch, "-O2", "-I", kdir, "-Xcompiler", "-fPIC", "-c", src, "-o", obj], check=True)
            objs.append(obj)
        os.makedirs(os.path.dirname(os.path.abspath(lib_path)), exist_ok=True)
        subprocess.run([nvcc, *arch, "-shared", "-o", lib_path, *objs], check=True)
    print(f"built {lib_path}")


# --------------------------------------------------------------------- the run
def run(lib_path: str, out_path: str) -> None:
    import torch

    lib = ctypes.CDLL(os.path.abspath(lib_path))
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    u, fl = ctypes.c_uint, ctypes.c_float
    out = {}

    def ok(rc, what):
        if rc != 0:
            raise RuntimeError(f"{what}: CUDA error {rc}")

    for case, (heads, rows, start, window) in PREFILL_CASES.items():
        nq, nkv, d = HEADS[heads]
        x = golden_inputs(case)
        q, k, v = dev(x["q"]), dev(x["k"]), dev(x["v"])
        scale = float(np.float32(1.0) / np.sqrt(np.float32(d)))
        keep_r, keep_h = kept_rows(rows, heads), kept_heads(heads)
        pick = lambda a: a[keep_r][:, keep_h]
        o = torch.zeros_like(q)
        ok(lib.gold_attention_prefill(ptr(q), ptr(k), ptr(v), ptr(o), u(nq), u(nkv), u(d), u(start), u(rows),
                                      u(window), fl(scale)), "attention_prefill_kernel")
        out[f"prefill/{case}"] = pick(o.cpu().numpy())
        # the online kernel, unsplit, and with its keys split over blocks where no window
        # narrows them (a block's range starts at max(split * split_len, window's start))
        for splits in sorted({1, ONLINE_SPLITS.get(case, 1)}):
            o = torch.zeros_like(q)
            part = torch.zeros(rows * nq * splits * (d + 2), dtype=torch.float32, device="cuda")
            ok(lib.gold_attention_online(ptr(q), ptr(k), ptr(v), ptr(o), ptr(part), u(nq), u(nkv), u(d), u(start),
                                         u(rows), u(window), u(splits), fl(scale)), "attention_online_kernel")
            out[f"online{splits}/{case}"] = pick(o.cpu().numpy())
        if window == 0:
            # the one-row kernel: the last query row over every position
            o = torch.zeros(nq, d, dtype=torch.float32, device="cuda")
            ok(lib.gold_attention(ptr(q[rows - 1].contiguous()), ptr(k), ptr(v), ptr(o), u(nq), u(nkv), u(d),
                                  u(start + rows), fl(scale)), "attention_kernel")
            out[f"decode/{case}"] = o.cpu().numpy()[keep_h]

    x = golden_inputs("gemv")
    xs, w = dev(x["x"]), dev(x["w"])
    y = torch.zeros(3, 1000, dtype=torch.float32, device="cuda")
    for r in range(3):
        ok(lib.gold_gemv(ptr(xs[r]), ptr(w), ptr(y[r]), u(96), u(1000)), "gemv_kernel")
    out["gemv"] = y.cpu().numpy()

    x = golden_inputs("rmsnorm")
    xs, w, b = dev(x["x"]), dev(x["w"]), dev(x["b"])
    o = torch.zeros_like(xs)
    ok(lib.gold_rmsnorm(ptr(xs), ptr(w), ptr(o), u(3), u(96), fl(1e-6)), "rmsnorm_kernel")
    out["rmsnorm"] = o.cpu().numpy()
    a, o = xs[1].clone(), torch.zeros(96, dtype=torch.float32, device="cuda")
    ok(lib.gold_add_rmsnorm(ptr(a), ptr(b[1].contiguous()), ptr(w), ptr(o), u(96), fl(1e-6)), "add_rmsnorm_kernel")
    out["add_rmsnorm/sum"], out["add_rmsnorm/out"] = a.cpu().numpy(), o.cpu().numpy()

    x = golden_inputs("pair")
    x1, w1, x2, w2 = (dev(x[n]) for n in ("x1", "w1", "x2", "w2"))
    o1, o2 = torch.zeros_like(x1), torch.zeros_like(x2)
    ok(lib.gold_rmsnorm_pair(ptr(x1), ptr(w1), ptr(o1), u(6), ptr(x2), ptr(w2), ptr(o2), u(2), u(32), fl(1e-5)),
       "rmsnorm_pair_kernel")
    out["pair/o1"], out["pair/o2"] = o1.cpu().numpy(), o2.cpu().numpy()

    t = dev(golden_inputs("rope")["t"])
    ok(lib.gold_rope_batch(ptr(t), u(100), u(6), u(32), u(32), u(17), fl(1e6)), "rope_batch_kernel")
    out["rope"] = t.cpu().numpy()

    np.savez_compressed(out_path, **out)
    total = sum(a.size for a in out.values())
    print(f"wrote {out_path}: {len(out)} arrays, {total} numbers")


if __name__ == "__main__":
    if len(sys.argv) == 4 and sys.argv[1] == "build":
        build(sys.argv[2], sys.argv[3])
    elif len(sys.argv) == 4 and sys.argv[1] == "run":
        run(sys.argv[2], sys.argv[3])
    else:
        print(__doc__)
        sys.exit(2)
