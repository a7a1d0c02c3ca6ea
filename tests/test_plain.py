"""The plain implementation checked against itself and against pinned outputs
of the reference's elementwise CUDA sources (no GPU)."""

import json
import math
import os

import numpy as np
import pytest

import plain_model as pm

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "elementwise_golden.json")


def test_rms_norm_properties():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(5, 48))
    y = pm.rms_norm(x, np.ones(48), 0.0)
    np.testing.assert_allclose(np.sqrt((y * y).mean(-1)), 1.0, rtol=1e-12)
    big = pm.rms_norm(x, np.ones(48), 1e6)
    assert np.abs(big).max() < 1e-2  # eps is added to the mean square


def test_rope_is_a_rotation_and_identity_at_zero():
    rng = np.random.default_rng(1)
    t = rng.normal(size=(4, 3, 32))
    pos = np.array([0, 1, 77, 4000])
    r = pm.rope_neox(t, pos, 1e4, 32)
    np.testing.assert_allclose(r[0], t[0], atol=1e-15)
    np.testing.assert_allclose((r * r).sum(-1), (t * t).sum(-1), rtol=1e-12)
    part = pm.rope_neox(t, pos, 1e4, 16)
    np.testing.assert_array_equal(part[..., 16:], t[..., 16:])
    # the dot product of two rotated vectors depends on the position difference only
    a, b = rng.normal(size=(1, 1, 32)), rng.normal(size=(1, 1, 32))
    d1 = (pm.rope_neox(a, np.array([10]), 1e4, 32) * pm.rope_neox(b, np.array([3]), 1e4, 32)).sum()
    d2 = (pm.rope_neox(a, np.array([107]), 1e4, 32) * pm.rope_neox(b, np.array([100]), 1e4, 32)).sum()
    assert abs(d1 - d2) < 1e-9


def test_attention_is_causal_grouped_and_windowed():
    rng = np.random.default_rng(2)
    T, nq, nkv, d = 12, 6, 2, 8
    q, k, v = rng.normal(size=(T, nq, d)), rng.normal(size=(T, nkv, d)), rng.normal(size=(T, nkv, d))
    full = pm.causal_attention(q, k, v, 0.3, None)
    np.testing.assert_allclose(full[0, 0], v[0, 0])  # the first query sees one key
    np.testing.assert_allclose(full[0, 5], v[0, 1])  # head 5 reads kv head 5 // 3
    cut = pm.causal_attention(q[:7], k[:7], v[:7], 0.3, None)
    np.testing.assert_allclose(cut, full[:7])  # later tokens change nothing earlier
    np.testing.assert_allclose(pm.causal_attention(q, k, v, 0.3, T), full)
    w1 = pm.causal_attention(q, k, v, 0.3, 1)
    np.testing.assert_allclose(w1[:, 0], v[:, 0])  # a window of 1 sees itself only
    w3 = pm.causal_attention(q, k, v, 0.3, 3)
    k2 = k.copy()
    k2[:5] += 100.0  # keys 0..4 are outside the window of query 7 (sees 5, 6, 7)
    np.testing.assert_allclose(pm.causal_attention(q, k2, v, 0.3, 3)[7], w3[7])


def test_forward_prefix_invariance():
    import helpers

    folder = helpers.model_folder("B", 7, "float32")
    cfg, w = pm.read_model(folder)
    toks = helpers.random_tokens(20, cfg["vocab_size"], 0)
    a = pm.forward(cfg, w, toks)
    b = pm.forward(cfg, w, toks[:9])
    np.testing.assert_allclose(a[:9], b, rtol=1e-10, atol=1e-12)
    assert a.shape == (20, cfg["vocab_size"])


def test_sampling_reference():
    l = np.array([0.0, 3.0, 3.0, -1.0], dtype=np.float32)
    assert pm.argmax_last(l) == 2  # ties: the highest index
    assert pm.sample_token(l, 1.0, 0.999, top_k=1) == 1  # a cut keeps the lowest index of a tie
    assert pm.sample_token(l, 1.0, 0.0) == 0
    assert pm.sample_token(l, 1.0, 0.9999999) == 3
    assert pm.sample_token(l, 1.0, 0.5, top_p=0.0) == 1
    # top_k=2 keeps ids 1 and 2: u below one half picks 1, above picks 2
    assert pm.sample_token(l, 1.0, 0.49, top_k=2) == 1
    assert pm.sample_token(l, 1.0, 0.51, top_k=2) == 2
    counts = np.zeros(4)
    for i in range(4000):
        counts[pm.sample_token(l, 0.7, (i + 0.5) / 4000)] += 1
    p = np.exp(l / 0.7)
    p /= p.sum()
    np.testing.assert_allclose(counts / 4000, p, atol=2e-3)


@pytest.mark.skipif(not os.path.exists(GOLDEN), reason="golden file absent")
def test_formulas_match_the_reference_sources():
    """Outputs of the reference's own rmsnorm_rms_inv, rope_kernel,
    silu_and_mul_kernel and add_kernel, compiled once for the CPU by
    tests/golden/make_elementwise_golden.py, against this file's functions."""
    with open(GOLDEN) as f:
        g = json.load(f)
    x = np.array(g["rmsnorm"]["x"], dtype=np.float64)
    inv = 1.0 / math.sqrt(float((x * x).mean()) + g["rmsnorm"]["eps"])
    assert abs(inv - g["rmsnorm"]["rms_inv"]) < 2e-6 * inv
    w = np.ones_like(x)
    np.testing.assert_allclose(pm.rms_norm(x, w, g["rmsnorm"]["eps"]), x * g["rmsnorm"]["rms_inv"], rtol=3e-6)
    for case in g["rope"]:
        t = np.array(case["x"], dtype=np.float64).reshape(1, case["heads"], case["head_dim"])
        got = pm.rope_neox(t, np.array([case["pos"]]), case["base"], case["rotary_dim"])
        np.testing.assert_allclose(got.reshape(-1), np.array(case["y"]), rtol=0, atol=case["atol"])
    s = g["silu_and_mul"]
    gate, up = np.array(s["gate"]), np.array(s["up"])
    # through the function the engine is held to: with x = [gate, up] and selector
    # matrices, pm.swiglu's products hand it exactly these gates and ups
    n = len(gate)
    eye, zero = np.eye(n), np.zeros((n, n))
    x = np.concatenate([gate, up])[None, :]
    got = pm.swiglu(x, np.hstack([eye, zero]), np.hstack([zero, eye]), eye)[0]
    np.testing.assert_allclose(got, np.array(s["y"]), rtol=2e-6, atol=1e-7)
    a = g["add"]
    np.testing.assert_allclose(np.array(a["a"]) + np.array(a["b"]), np.array(a["y"]), rtol=1e-7)


# ----------------------------------------------------------- the 32-bit mirror
def test_mirror_exponential_and_sine_cosine_are_accurate():
    """The mirror's own exp and sin/cos (IEEE operations only) against NumPy in
    double: a few units in the last place at most, over the ranges the model
    uses (softmax and SiLU arguments; angles up to a long context's position)."""
    import fp32_mirror as mir

    rng = np.random.default_rng(0)
    xs = np.concatenate([rng.uniform(-90, 88.7, 4000), rng.uniform(-1, 1, 2000), [0.0, -0.0, 88.7, -87.3, -103.0]])
    for x in xs.astype(np.float32):
        got, ref = mir.exp(float(x)), math.exp(float(x))
        assert abs(got - ref) <= 3 * np.spacing(np.float32(ref)), (x, got, ref)
    assert mir.exp(float("-inf")) == 0.0 and mir.exp(-200.0) == 0.0 and mir.exp(100.0) == float("inf")
    assert math.isnan(mir.exp(float("nan")))
    assert 0.0 < mir.exp(-100.0) < 1e-43  # a subnormal result
    for t in np.concatenate([rng.uniform(-10, 10, 2000), rng.uniform(0, 1e5, 3000), [0.0, 40959.0, 1.0e7]]).astype(np.float32):
        s, c = mir.sincos(float(t))
        assert abs(s - math.sin(float(t))) <= 6.1e-8 and abs(c - math.cos(float(t))) <= 6.1e-8, t


def test_mirror_agrees_with_the_plain_model_and_sees_a_changed_order():
    """The mirror follows the same formulas as the float64 plain model (so it is
    within 32-bit rounding of it), and a change of one reduction order (the
    norm's sum of squares in plain index order) changes its bits: a bit-for-bit
    comparison with it therefore sees such a change in a kernel."""
    import fp32_mirror as mir
    import helpers

    for name in ("A", "B"):
        folder = helpers.model_folder(name, 7, "float32")
        cfg, w = pm.read_model(folder)
        toks = helpers.random_tokens(40, cfg["vocab_size"], 1)
        ref = pm.forward(cfg, w, toks)
        got = mir.forward(cfg, w, toks)
        assert got.dtype == np.float32 and got.shape == ref.shape
        assert helpers.rel_err(got, ref) < 3e-6
        other = mir.forward(cfg, w, toks, norm_order=1)
        assert helpers.rel_err(other, ref) < 3e-6
        assert not np.array_equal(got, other)
    # each part alone against its plain form
    rng = np.random.default_rng(3)
    T, nq, nkv, d = 9, 6, 2, 48
    q, k, v = (rng.normal(size=(T, n, d)).astype(np.float32) for n in (nq, nkv, nkv))
    a = mir.attention(q, k, v, 0.2, 4)
    np.testing.assert_allclose(a, pm.causal_attention(q.astype(np.float64), k.astype(np.float64), v.astype(np.float64), 0.2, 4),
                               rtol=2e-5, atol=2e-6)
    wn = (1 + 0.1 * rng.normal(size=d)).astype(np.float32)
    pos = np.array([0, 1, 5, 63, 64, 200, 999, 4095, 40000])
    got = mir.head_norm_rope(q, wn, 1e-6, mir.rope_denominators(1e4, 32), 32, pos)
    ref = pm.rope_neox(pm.rms_norm(q.astype(np.float64), wn.astype(np.float64), 1e-6), pos, 1e4, 32)
    np.testing.assert_allclose(got, ref, rtol=0, atol=5e-3)  # the 32-bit angle is off by up to pos * 2^-24
    np.testing.assert_allclose(got[:3], ref[:3], rtol=0, atol=2e-6)  # positions 0, 1, 5


# ------------------------------------ the reference's own kernels, run once on a GPU
KERNEL_GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "kernel_golden.npz")


@pytest.mark.skipif(not os.path.exists(KERNEL_GOLDEN), reason="golden file absent")
def test_plain_parts_match_the_reference_kernels_outputs():
    """Outputs of the reference's attention_kernel, attention_prefill_kernel,
    attention_online_kernel (+ combine), gemv_kernel, rmsnorm_kernel,
    add_rmsnorm_kernel, rmsnorm_pair_kernel and rope_batch_kernel, compiled
    unchanged from its checkout and run once on a GPU by
    tests/golden/make_kernel_golden.py, against this folder's plain functions on
    the same inputs (rebuilt from the seeds): the scale, the causal and window
    bounds, the head map h // group, the softmax, x W^T, the norm with and
    without the add before it, the rotation.  The bound for attention is the
    reference's own between its kernels (1e-5,
    src/model/attention_online_tests.rs:14); the 32-bit mirror is held to the
    same numbers."""
    sys_path_golden = os.path.join(os.path.dirname(__file__), "golden")
    import sys

    sys.path.insert(0, sys_path_golden)
    try:
        import make_kernel_golden as mk
    finally:
        sys.path.remove(sys_path_golden)
    import fp32_mirror as mir

    g = np.load(KERNEL_GOLDEN)
    D = np.float64
    for case, (heads, rows, start, window) in mk.PREFILL_CASES.items():
        nq, nkv, d = mk.HEADS[heads]
        x = mk.golden_inputs(case)
        scale = float(np.float32(1.0) / np.sqrt(np.float32(d)))
        keep_r, keep_h = mk.kept_rows(rows, heads), mk.kept_heads(heads)
        T = start + rows
        qfull = np.zeros((T, nq, d), dtype=D)
        qfull[start:] = x["q"]
        ref = pm.causal_attention(qfull, x["k"].astype(D), x["v"].astype(D), scale, window or None,
                                  first_row=start)[start:]
        want = ref[keep_r][:, keep_h]
        for kind in ("prefill", "online1", f"online{mk.ONLINE_SPLITS.get(case, 1)}"):
            np.testing.assert_allclose(g[f"{kind}/{case}"], want, rtol=0, atol=1e-5, err_msg=f"{kind}/{case}")
        if f"decode/{case}" in g.files:
            np.testing.assert_allclose(g[f"decode/{case}"], ref[rows - 1][keep_h], rtol=0, atol=1e-5)
        # the mirror of the 32-bit kernel, on the same case
        qm = np.zeros((T, nq, d), dtype=np.float32)
        qm[start:] = x["q"]
        got = mir.attention(qm, x["k"], x["v"], scale, window or None)[start:][keep_r][:, keep_h]
        np.testing.assert_allclose(got, g[f"prefill/{case}"], rtol=0, atol=1e-5)

    x = mk.golden_inputs("gemv")
    np.testing.assert_allclose(x["x"].astype(D) @ x["w"].astype(D).T, g["gemv"], rtol=0, atol=2e-6)
    np.testing.assert_allclose(mir.linear(x["x"], x["w"]), g["gemv"], rtol=0, atol=2e-6)

    x = mk.golden_inputs("rmsnorm")
    np.testing.assert_allclose(pm.rms_norm(x["x"].astype(D), x["w"].astype(D), 1e-6), g["rmsnorm"], rtol=3e-6, atol=1e-7)
    s = x["x"][1].astype(D) + x["b"][1].astype(D)  # add, then norm (src/kernels_cuda/decode_ops.cu:10-35)
    np.testing.assert_allclose(s, g["add_rmsnorm/sum"], rtol=2e-7, atol=1e-7)
    np.testing.assert_allclose(pm.rms_norm(s, x["w"].astype(D), 1e-6), g["add_rmsnorm/out"], rtol=3e-6, atol=1e-7)
    out, t = mir.rms_norm(x["x"][1:2], x["w"], 1e-6, delta=x["b"][1:2])
    assert np.array_equal(t[0], g["add_rmsnorm/sum"])
    np.testing.assert_allclose(out[0], g["add_rmsnorm/out"], rtol=3e-6, atol=1e-7)

    x = mk.golden_inputs("pair")  # the per-head q and k norms: one weight vector for all heads
    np.testing.assert_allclose(pm.rms_norm(x["x1"].astype(D), x["w1"].astype(D), 1e-5), g["pair/o1"], rtol=3e-6, atol=1e-7)
    np.testing.assert_allclose(pm.rms_norm(x["x2"].astype(D), x["w2"].astype(D), 1e-5), g["pair/o2"], rtol=3e-6, atol=1e-7)

    t = mk.golden_inputs("rope")["t"]
    pos = np.arange(100, 117)
    # the reference's angle is 32-bit (position / powf(base, e)): off from double by up to position * 2^-24
    np.testing.assert_allclose(pm.rope_neox(t.astype(D), pos, 1e6, 32), g["rope"], rtol=0, atol=5e-5)
    got = mir.head_norm_rope(t, None, 0.0, mir.rope_denominators(1e6, 32), 32, pos)
    np.testing.assert_allclose(got, g["rope"], rtol=0, atol=5e-5)
