"""A plain, slow implementation of the Qwen3 dense forward pass, for tests.

Whole sequences, no cache, one function per part, NumPy in double precision;
it shares no code with `reflex_b200`.  The reference's model code is Rust over
CUDA (no Rust toolchain here, and it needs a GPU and a GGUF file), so it cannot
be imported or compiled on this machine's CPU: this file rests on the
reference's formulas, cited function by function, and on its elementwise CUDA
sources, against which `tests/golden/` pins the norm, rotary, SiLU and add
formulas once.
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np

F = np.float64


# --------------------------------------------------------------------- files
def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    """name -> float64 array (bfloat16 and float32 are widened exactly)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        blob = f.read()
    out = {}
    for name, ent in header.items():
        if name == "__metadata__":
            continue
        b, e = ent["data_offsets"]
        raw = blob[b:e]
        shape = ent["shape"]
        if ent["dtype"] == "BF16":
            u16 = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u16.view(np.float32)
        elif ent["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4")
        elif ent["dtype"] == "F16":
            arr = np.frombuffer(raw, dtype="<f2")
        else:
            raise ValueError(f"plain reader: dtype {ent['dtype']} of {name}")
        out[name] = arr.astype(F).reshape(shape)
    return out


def read_model(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# --------------------------------------------------------------------- parts
def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """y = (x * r) * w, r = 1/sqrt(mean(x^2) + eps), over the last axis.
    src/kernels_cuda/rmsnorm.cuh:14-40 (r), src/kernels_cuda/rmsnorm.cu:44-52 (y)."""
    r = 1.0 / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return (x * r) * w


def rope_neox(t: np.ndarray, positions: np.ndarray, theta_base: float, rotary_dim: int) -> np.ndarray:
    """t: [T, heads, d].  Pairs (i, i + rd/2), i < rd/2:
    theta = pos / base^(2i/rd); (a, b) <- (a cos - b sin, a sin + b cos);
    elements >= rd untouched.  src/kernels_cuda/rope.cu:9-37."""
    half = rotary_dim // 2
    i = np.arange(half, dtype=F)
    denom = np.power(F(theta_base), 2.0 * i / rotary_dim)
    ang = positions.astype(F)[:, None] / denom[None, :]  # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = t.copy()
    a, b = t[..., :half], t[..., half:rotary_dim]
    out[..., :half] = a * c - b * s
    out[..., half:rotary_dim] = a * s + b * c
    return out


def causal_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float,
                     window: Optional[int], first_row: int = 0) -> np.ndarray:
    """q: [T, nq, d], k, v: [T, nkv, d] of one whole sequence.  Query i of head h
    reads kv head h // (nq/nkv) (src/kernels_cuda/attention_online.cuh:56) and
    keys j <= i, with a window only those with i - j < window
    (src/model/config.rs:1184-1185); s_j = (q . k_j) * scale, softmax with the
    maximum subtracted, out = sum_j p_j v_j
    (plain form: src/kernels_cuda/attention.cu:36-74).  Rows before `first_row`
    are left zero (tests that need only a sequence's last rows skip the rest)."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    g = nq // nkv
    out = np.zeros_like(q)
    for h in range(nq):
        kh = h // g
        for i in range(first_row, T):
            lo = 0 if not window else max(0, i - window + 1)
            s = (k[lo:i + 1, kh, :] @ q[i, h, :]) * scale
            p = np.exp(s - s.max())
            out[i, h, :] = (p[:, None] * v[lo:i + 1, kh, :]).sum(axis=0) / p.sum()
    return out


def swiglu(x: np.ndarray, wg: np.ndarray, wu: np.ndarray, wd: np.ndarray) -> np.ndarray:
    """down(silu(gate) * up), silu(g) = g / (1 + exp(-g)); linear layers are
    y = x W^T with W [out, in].  src/model/dense.rs:1476-1481,
    src/kernels_cuda/silu_and_mul.cu:7-23."""
    g = x @ wg.T
    u = x @ wu.T
    return ((g / (1.0 + np.exp(-g))) * u) @ wd.T


def layer_windows(cfg: dict) -> List[Optional[int]]:
    n = cfg["num_hidden_layers"]
    types = cfg.get("layer_types")
    if types is None:
        if cfg.get("use_sliding_window") and cfg.get("sliding_window") is not None:
            first = cfg.get("max_window_layers", n)
            types = ["sliding_attention" if i >= first else "full_attention" for i in range(n)]
        else:
            types = ["full_attention"] * n
    return [cfg.get("sliding_window") if t == "sliding_attention" else None for t in types]


def decoder_layer(h: np.ndarray, w: Dict[str, np.ndarray], prefix: str, cfg: dict,
                  positions: np.ndarray, window: Optional[int]) -> np.ndarray:
    """Pre-norm block: norm -> q,k,v -> per-head q/k norm -> rotary -> attention
    -> o -> add; norm -> SwiGLU -> add.  src/model/dense.rs:1337-1431, 1469-1481."""
    nq, nkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // nq
    eps = cfg["rms_norm_eps"]
    T = h.shape[0]
    x = rms_norm(h, w[prefix + "input_layernorm.weight"], eps)
    q = (x @ w[prefix + "self_attn.q_proj.weight"].T).reshape(T, nq, d)
    k = (x @ w[prefix + "self_attn.k_proj.weight"].T).reshape(T, nkv, d)
    v = (x @ w[prefix + "self_attn.v_proj.weight"].T).reshape(T, nkv, d)
    q = rms_norm(q, w[prefix + "self_attn.q_norm.weight"], eps)  # one weight for all heads
    k = rms_norm(k, w[prefix + "self_attn.k_norm.weight"], eps)
    q = rope_neox(q, positions, cfg["rope_theta"], d)
    k = rope_neox(k, positions, cfg["rope_theta"], d)
    a = causal_attention(q, k, v, 1.0 / math.sqrt(d), window).reshape(T, nq * d)
    h = h + a @ w[prefix + "self_attn.o_proj.weight"].T
    x = rms_norm(h, w[prefix + "post_attention_layernorm.weight"], eps)
    h = h + swiglu(x, w[prefix + "mlp.gate_proj.weight"], w[prefix + "mlp.up_proj.weight"],
                   w[prefix + "mlp.down_proj.weight"])
    return h


def forward(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int]) -> np.ndarray:
    """Logits [T, vocab] of one whole sequence.  Embedding rows unscaled
    (src/model/dense.rs:1959-1967); final norm then head, tied to the embedding
    when the model has no head of its own (src/model/mod.rs:1191-1202,
    src/model/dense.rs:661-697)."""
    tokens = np.asarray(tokens, dtype=np.int64)
    positions = np.arange(len(tokens))
    h = w["model.embed_tokens.weight"][tokens].astype(F)
    windows = layer_windows(cfg)
    for i in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, w, f"model.layers.{i}.", cfg, positions, windows[i])
    x = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return x @ head.T


# ------------------------------------------------------------------ sampling
def argmax_last(logits: np.ndarray) -> int:
    """Greedy choice; ties go to the highest index (src/model/mod.rs:1371-1380)."""
    m = logits.max()
    return int(np.nonzero(logits == m)[0][-1])


def sample_token(logits: np.ndarray, temperature: float, u: float,
                 top_k: Optional[int] = None, top_p: Optional[float] = None) -> int:
    """Temperature softmax, top-k, top-p, inverse-CDF draw with the uniform `u`
    (src/sampling.rs:241-294).  Ties at a cut are kept lowest index first and the
    draw walks the kept entries in index order."""
    l = logits.astype(np.float32)
    p = np.exp((l - l.max()) / np.float32(temperature)).astype(np.float32)
    total = p.sum(dtype=np.float32)
    order = np.lexsort((np.arange(len(p)), -p))  # descending p, then ascending index
    n_keep = len(p)
    if top_k is not None and 0 < top_k < len(p):
        n_keep = top_k
    if top_p is not None and top_p < 1.0:
        cum = np.cumsum(p[order] / total, dtype=np.float64)
        n_p = int(np.searchsorted(cum, top_p, side="left")) + 1
        n_keep = min(n_keep, max(1, n_p))
    kept = np.zeros(len(p), dtype=bool)
    kept[order[:n_keep]] = True
    renorm = p[kept].sum(dtype=np.float64)
    draw = u * renorm
    acc = 0.0
    last = 0
    for i in np.nonzero(kept)[0]:
        acc += float(p[i])
        last = int(i)
        if draw <= acc:
            return int(i)
    return last
