"""The Python side of the C interface: plain functions over plain values
(ints, floats, lists, bytes) that `engine_abi.cpp` calls.  Nothing here is
meant for Python callers, who have `reflex_b200.Model`.
"""

from __future__ import annotations

import json
import os
from typing import List, Optional, Sequence, Tuple

from ..errors import InvalidInput, IoError, ReflexError


def describe_error(exc: BaseException) -> Tuple[int, str]:
    """(stable category number, message) of an exception."""
    if isinstance(exc, ReflexError):
        return int(exc.code), str(exc)
    if isinstance(exc, FileNotFoundError):
        return IoError.code, str(exc)
    if isinstance(exc, MemoryError):
        return 5, str(exc) or "out of memory"
    if isinstance(exc, OSError):
        return IoError.code, str(exc)
    return 12, f"{type(exc).__name__}: {exc}"


def _kwargs(max_tokens: int, max_batch: int) -> dict:
    kw = {}
    if max_tokens > 0:
        kw["max_tokens"] = int(max_tokens)
    if max_batch > 0:
        kw["max_batch"] = int(max_batch)
    return kw


def load(model_dir: str, weights: str, max_tokens: int, max_batch: int):
    from ..api import Model

    if not os.path.isdir(model_dir):
        raise IoError(f"{model_dir}: no such model folder")
    return Model.load(model_dir, weights=weights or "bf16", **_kwargs(max_tokens, max_batch))


def load_random(config_json: str, seed: int, out_dir: str, weights: str, max_tokens: int, max_batch: int):
    from ..weights import write_random_model

    try:
        with open(config_json, "r", encoding="utf-8") as f:
            cfg = json.load(f)
    except FileNotFoundError as e:
        raise IoError(f"{config_json}: no such file") from e
    dtype = "float32" if (weights or "bf16") in ("f32", "float32", "fp32") else "bfloat16"
    write_random_model(cfg, int(seed), out_dir, dtype)
    return load(out_dir, weights, max_tokens, max_batch)


def generate(model, prompts: List[List[int]], max_new_tokens: int, temperature: float, top_k: int,
             top_p: float, seed: int, stop_ids: Sequence[int]) -> List[List[int]]:
    from ..sampling import SamplingParams

    params = SamplingParams(
        temperature=float(temperature),
        top_k=int(top_k) if top_k > 0 else None,
        top_p=float(top_p) if 0.0 < top_p < 1.0 else None,
        seed=int(seed) if seed >= 0 else None,
        stop_token_ids=tuple(int(t) for t in stop_ids),
    )
    if len(prompts) == 0:
        raise InvalidInput("no prompts")
    return [list(map(int, seq)) for seq in model.generate([list(p) for p in prompts], int(max_new_tokens), params)]


def score(model, prompt: List[int], candidates: List[List[int]], temperature: float):
    resp = model.system1_evaluate(prompt, candidates, float(temperature))
    return ([float(r.score) for r in resp.results], [float(p) for p in resp.probabilities],
            int(resp.best_idx), float(resp.entropy))


def open_sequence(model) -> int:
    return int(model.engine.open())


def close_sequence(model, sequence: int) -> None:
    model.engine.close(int(sequence))


def step(model, entries: List[Tuple[int, List[int], List[int]]]) -> Tuple[int, int, Optional[bytes]]:
    """(rows, vocab, little-endian float32 bytes of the wanted logits)."""
    logits = model.engine.step([(int(s), list(t), list(w)) for s, t, w in entries])
    vocab = int(model.spec.vocab_size)
    if logits is None or logits.numel() == 0:
        return 0, vocab, None
    host = logits.float().contiguous().cpu()
    return int(host.shape[0]), vocab, host.numpy().tobytes()
