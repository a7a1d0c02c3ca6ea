"""Shared test helpers: tiny model folders, replay schedules, comparisons."""

from __future__ import annotations

import os
import tempfile
from typing import Dict, List, Sequence, Tuple

import numpy as np

import plain_model
from tiny_configs import ALL

_FOLDERS: Dict[Tuple[str, int, str, float, str], str] = {}
_PLAIN_CACHE: Dict[Tuple[str, Tuple[int, ...]], np.ndarray] = {}


def model_folder(name: str, seed: int = 7, dtype: str = "float32", sharp: float = 1.0,
                 sharp_layers: str = "all") -> str:
    """A model folder with random weights in a temporary place (made once).

    Random N(0, 0.02) weights give nearly flat attention, which would hide a
    missing or misplaced key (each key moves the output by about 1/n).  With
    `sharp` > 1 the per-head q and k norm weights are scaled so that scores
    spread by about sharp^2 and a few keys dominate each softmax; in all
    layers, or (`sharp_layers="last"`) in the last layer only.  A peaked
    softmax multiplies an upstream relative error by about the scores' spread,
    layer after layer, so rounding noise grows quickly when all layers are
    sharp: fine in float32, too much in bfloat16, where only the last layer is
    sharpened."""
    import torch

    from reflex_b200.weights import SafetensorsFile, write_random_model, write_safetensors

    key = (name, seed, dtype, sharp, sharp_layers)
    if key not in _FOLDERS:
        d = tempfile.mkdtemp(prefix=f"rfx_tiny_{name}_")
        write_random_model(ALL[name], seed, d, dtype)
        if sharp != 1.0:
            path = os.path.join(d, "model.safetensors")
            f = SafetensorsFile(path)
            tensors = [(k, f.tensor(k).clone()) for k in f.keys()]
            f.close()
            last = f"model.layers.{ALL[name]['num_hidden_layers'] - 1}."

            def hit(k):
                return k.endswith(("q_norm.weight", "k_norm.weight")) and (
                    sharp_layers == "all" or k.startswith(last))

            tensors = [(k, (t.float() * sharp).to(t.dtype)) if hit(k) else (k, t) for k, t in tensors]
            write_safetensors(path, tensors)
        _FOLDERS[key] = d
    return _FOLDERS[key]


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, vocab, size=n)]


def plain_logits(folder: str, tokens: Sequence[int]) -> np.ndarray:
    key = (folder, tuple(tokens))
    if key not in _PLAIN_CACHE:
        cfg, w = plain_model.read_model(folder)
        _PLAIN_CACHE[key] = plain_model.forward(cfg, w, tokens)
    return _PLAIN_CACHE[key]


def make_engine(folder: str, dtype: str, max_tokens: int = 4096, **kw):
    import torch

    import reflex_b200
    from reflex_b200.engine import Engine

    model = reflex_b200.load_model(folder, dtype, "cuda:0")
    return Engine(model, max_tokens=max_tokens, **kw)


def rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    """max |got - ref| / max |ref|: logits of random tiny models are small, so
    the error is measured against their scale."""
    return float(np.abs(got.astype(np.float64) - ref).max() / np.abs(ref).max())


def run_whole(engine, tokens: Sequence[int]) -> np.ndarray:
    s = engine.open()
    out = engine.step([(s, tokens, list(range(len(tokens))))]).float().cpu().numpy()
    engine.close(s)
    return out


def run_tail_one_by_one(engine, tokens: Sequence[int], tail: int = 32) -> np.ndarray:
    """First len - tail tokens in one step, the rest one token a step."""
    n = len(tokens)
    head = max(1, n - tail)
    s = engine.open()
    outs = [engine.step([(s, tokens[:head], list(range(head)))]).float().cpu().numpy()]
    for i in range(head, n):
        outs.append(engine.step([(s, [tokens[i]], [0])]).float().cpu().numpy())
    engine.close(s)
    return np.concatenate(outs, axis=0)


def run_batches(engine, requests: List[Sequence[int]], batch_size: int, prefill: Sequence[int]) -> List[np.ndarray]:
    """Requests in batches of `batch_size`, one batch after another.  In a batch
    request i brings its first prefill[i % len] tokens (at most its length) in
    step 0, then one token a step until it is out of tokens; shorter requests
    end earlier and give their slots back.  Returns per-request logits at every
    position."""
    results: List[np.ndarray] = [None] * len(requests)
    for b0 in range(0, len(requests), batch_size):
        idx = list(range(b0, min(len(requests), b0 + batch_size)))
        seqs = {i: engine.open() for i in idx}
        fed = {i: 0 for i in idx}
        chunks = {i: [] for i in idx}
        first = True
        while seqs:
            entries, order = [], []
            for i in list(seqs):
                toks = requests[i]
                if first:
                    n = min(len(toks), max(1, prefill[i % len(prefill)]))
                else:
                    n = 1
                part = toks[fed[i]:fed[i] + n]
                entries.append((seqs[i], part, list(range(len(part)))))
                order.append((i, len(part)))
            out = engine.step(entries).float().cpu().numpy()
            r = 0
            for i, n in order:
                chunks[i].append(out[r:r + n])
                r += n
                fed[i] += n
                if fed[i] >= len(requests[i]):
                    engine.close(seqs.pop(i))
                    results[i] = np.concatenate(chunks[i], axis=0)
            first = False
    return results
