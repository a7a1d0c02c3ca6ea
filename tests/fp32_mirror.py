"""The host mirror of the true 32-bit path: the model in float32, operation by
operation in the kernels' order, so that the engine's float32 logits can be
compared with it bit for bit.

The arithmetic is C++ (`tests/mirror/fp32_mirror.cpp`, one function per part,
built here by g++ with -ffp-contract=off at first use); this file wires the
parts into the Qwen3 dense model exactly as `plain_model.forward` does, whole
sequences and no cache.  `plain_model` (float64 NumPy) stays the independent
oracle: it says the formulas are right, the mirror says the 32-bit path
computes exactly what it claims, whatever the batch.  The reference anchors a
kernel the same way (src/model/rmsnorm_tests.rs:17-29, 64-72).
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import subprocess
import tempfile
from typing import Dict, Optional, Sequence

import numpy as np

import plain_model

_SRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mirror", "fp32_mirror.cpp")
_LIB: Optional[ctypes.CDLL] = None

F = np.float32
_fp = ctypes.POINTER(ctypes.c_float)
_ip = ctypes.POINTER(ctypes.c_int)


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        with open(_SRC, "rb") as f:
            tag = hashlib.sha256(f.read()).hexdigest()[:16]
        out = os.path.join(tempfile.gettempdir(), f"rfx_fp32_mirror_{os.getuid()}_{tag}.so")
        if not os.path.exists(out):
            tmp = out + f".{os.getpid()}"
            subprocess.run(["g++", "-O2", "-ffp-contract=off", "-shared", "-fPIC", "-o", tmp, _SRC], check=True)
            os.replace(tmp, out)
        _LIB = ctypes.CDLL(out)
        _LIB.mir_exp.argtypes = [ctypes.c_float]
        _LIB.mir_exp.restype = ctypes.c_float
        _LIB.mir_sincos.argtypes = [ctypes.c_float, _fp, _fp]
        _LIB.mir_sincos.restype = None
    return _LIB


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(_fp)


def _f(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=F)


def exp(x: float) -> float:
    return float(lib().mir_exp(ctypes.c_float(x)))


def sincos(theta: float):
    s, c = ctypes.c_float(), ctypes.c_float()
    lib().mir_sincos(ctypes.c_float(theta), ctypes.byref(s), ctypes.byref(c))
    return s.value, c.value


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float, delta: Optional[np.ndarray] = None,
             w_offset: float = 0.0, order: int = 0):
    """(normed rows, x + delta)."""
    x = _f(x)
    R, H = x.shape
    d = None if delta is None else _f(delta)
    t, out = np.empty_like(x), np.empty_like(x)
    lib().mir_rmsnorm(_p(x), _p(d), _p(t), _p(_f(w)), ctypes.c_float(eps), ctypes.c_float(w_offset),
                      _p(out), R, H, order)
    return out, t


def linear(x: np.ndarray, W: np.ndarray) -> np.ndarray:
    x, W = _f(x), _f(W)
    R, K = x.shape
    N = W.shape[0]
    y = np.empty((R, N), dtype=F)
    lib().mir_linear(_p(x), _p(W), _p(y), R, N, K)
    return y


def head_norm_rope(heads: np.ndarray, w: Optional[np.ndarray], eps: float, denom: Optional[np.ndarray],
                   rotary_dim: int, positions: Sequence[int], pairing: int = 0, magnitude: float = 1.0,
                   w_offset: float = 0.0) -> np.ndarray:
    """heads [T, n, d] -> per-head norm (if w) and rotation, a new array."""
    out = _f(heads).copy()
    T, n, d = out.shape
    pos = np.ascontiguousarray(positions, dtype=np.int32)
    lib().mir_head_norm_rope(_p(out), _p(None if w is None else _f(w)), ctypes.c_float(eps),
                             ctypes.c_float(w_offset), _p(None if denom is None else _f(denom)), rotary_dim,
                             pairing, ctypes.c_float(magnitude), pos.ctypes.data_as(_ip), T, n, d)
    return out


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, window: Optional[int]) -> np.ndarray:
    q, k, v = _f(q), _f(k), _f(v)
    T, nq, d = q.shape
    out = np.empty_like(q)
    lib().mir_attention(_p(q), _p(k), _p(v), _p(out), T, nq, k.shape[1], d, int(window or 0),
                        ctypes.c_float(scale))
    return out


def swiglu_act(g: np.ndarray, u: np.ndarray) -> np.ndarray:
    g, u = _f(g), _f(u)
    out = np.empty_like(g)
    lib().mir_swiglu(_p(g), _p(u), _p(out), ctypes.c_longlong(g.size))
    return out


def rope_denominators(theta: float, rotary_dim: int) -> np.ndarray:
    """base^(2i/rd) in double, rounded to float32: the table the position part owns."""
    import math

    return np.array([math.pow(float(theta), 2.0 * i / float(rotary_dim)) for i in range(rotary_dim // 2)],
                    dtype=np.float64).astype(F)


def forward(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int], norm_order: int = 0) -> np.ndarray:
    """float32 logits [T, vocab] of one whole sequence.  `w` as `plain_model.read_model`
    gives it (float64 arrays holding float32 or bfloat16 values exactly)."""
    nq = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nq
    d = cfg.get("head_dim") or cfg["hidden_size"] // nq
    eps = cfg["rms_norm_eps"]
    T = len(tokens)
    positions = np.arange(T, dtype=np.int32)
    denom = rope_denominators(cfg["rope_theta"], d)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(d)))  # 1 / sqrtf((float) d)
    windows = plain_model.layer_windows(cfg)
    h = _f(w["model.embed_tokens.weight"][np.asarray(tokens, dtype=np.int64)])
    pending = None
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        x, h = rms_norm(h, w[p + "input_layernorm.weight"], eps, delta=pending, order=norm_order)
        q = linear(x, w[p + "self_attn.q_proj.weight"]).reshape(T, nq, d)
        k = linear(x, w[p + "self_attn.k_proj.weight"]).reshape(T, nkv, d)
        v = linear(x, w[p + "self_attn.v_proj.weight"]).reshape(T, nkv, d)
        q = head_norm_rope(q, w[p + "self_attn.q_norm.weight"], eps, denom, d, positions)
        k = head_norm_rope(k, w[p + "self_attn.k_norm.weight"], eps, denom, d, positions)
        a = attention(q, k, v, scale, windows[i]).reshape(T, nq * d)
        o = linear(a, w[p + "self_attn.o_proj.weight"])
        x, h = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps, delta=o, order=norm_order)
        act = swiglu_act(linear(x, w[p + "mlp.gate_proj.weight"]), linear(x, w[p + "mlp.up_proj.weight"]))
        pending = linear(act, w[p + "mlp.down_proj.weight"])
    x, _ = rms_norm(h, w["model.norm.weight"], eps, delta=pending, order=norm_order)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return linear(x, head)
