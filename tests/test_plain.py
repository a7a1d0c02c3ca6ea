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
    np.testing.assert_allclose((gate / (1.0 + np.exp(-gate))) * up, np.array(s["y"]), rtol=2e-6, atol=1e-7)
    a = g["add"]
    np.testing.assert_allclose(np.array(a["a"]) + np.array(a["b"]), np.array(a["y"]), rtol=1e-7)
