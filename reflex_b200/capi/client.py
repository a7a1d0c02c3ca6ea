"""A Python entry point over the C interface, through ctypes.

`reflex_b200.h` is what a C or C++ program links against; this module is the
same interface seen from Python, call for call (`rfx_load`, `rfx_generate`,
`rfx_score`, `rfx_open_sequence` / `rfx_step` / `rfx_close_sequence`,
`rfx_free*`, `rfx_last_error[_code]`), with failures turned back into the
library's exceptions by their stable category numbers.  The reference tells
Python users to drive its server instead (README.md:165-166); its C interface
is include/reflex_engine.h, whose rules (status codes, a thread-local last
error, library-owned result buffers with NULL-safe frees) the calls below rely
on.  `reflex_b200.Model` is the direct way in from Python; this one is for
programs that want to stay on the C interface's contract.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_uint64, c_void_p
from typing import List, Optional, Sequence, Tuple

from .. import errors


class _Sampling(Structure):
    _fields_ = [("temperature", c_float), ("top_k", c_int32), ("top_p", c_float), ("seed", c_int64),
                ("stop_token_ids", POINTER(c_uint32)), ("num_stop_token_ids", c_size_t)]


class _Sequence(Structure):
    _fields_ = [("token_ids", POINTER(c_uint32)), ("num_tokens", c_size_t)]


class _GenerateResult(Structure):
    _fields_ = [("sequences", POINTER(_Sequence)), ("num_sequences", c_size_t)]


class _CandidateScore(Structure):
    _fields_ = [("score", c_float), ("probability", c_float)]


class _ScoreResult(Structure):
    _fields_ = [("candidates", POINTER(_CandidateScore)), ("num_candidates", c_size_t),
                ("best_idx", c_size_t), ("entropy", c_float)]


class _StepResult(Structure):
    _fields_ = [("logits", POINTER(c_float)), ("rows", c_size_t), ("vocab", c_size_t)]


class _StepEntry(Structure):
    _fields_ = [("sequence", c_int64), ("tokens", POINTER(c_uint32)), ("num_tokens", c_size_t),
                ("want", POINTER(c_uint32)), ("num_want", c_size_t)]


_LIB: Optional[ctypes.CDLL] = None


def _lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        from . import build

        lib = ctypes.CDLL(build.ensure_built())
        lib.rfx_last_error.restype = c_char_p
        lib.rfx_last_error_code.restype = c_int
        lib.rfx_load.restype = c_void_p
        lib.rfx_load.argtypes = [c_char_p, c_char_p, c_size_t, c_size_t]
        lib.rfx_load_random.restype = c_void_p
        lib.rfx_load_random.argtypes = [c_char_p, c_uint64, c_char_p, c_char_p, c_size_t, c_size_t]
        lib.rfx_free.argtypes = [c_void_p]
        lib.rfx_generate.argtypes = [c_void_p, POINTER(POINTER(c_uint32)), POINTER(c_size_t), c_size_t, c_size_t,
                                     POINTER(_Sampling), POINTER(_GenerateResult)]
        lib.rfx_free_generate_result.argtypes = [POINTER(_GenerateResult)]
        lib.rfx_score.argtypes = [c_void_p, POINTER(c_uint32), c_size_t, POINTER(POINTER(c_uint32)),
                                  POINTER(c_size_t), c_size_t, c_float, POINTER(_ScoreResult)]
        lib.rfx_free_score_result.argtypes = [POINTER(_ScoreResult)]
        lib.rfx_open_sequence.argtypes = [c_void_p, POINTER(c_int64)]
        lib.rfx_close_sequence.argtypes = [c_void_p, c_int64]
        lib.rfx_step.argtypes = [c_void_p, POINTER(_StepEntry), c_size_t, POINTER(_StepResult)]
        lib.rfx_free_step_result.argtypes = [POINTER(_StepResult)]
        _LIB = lib
    return _LIB


def _by_code() -> dict:
    out = {}
    for name in dir(errors):
        cls = getattr(errors, name)
        if isinstance(cls, type) and issubclass(cls, errors.ReflexError) and getattr(cls, "code", None) is not None:
            out.setdefault(int(cls.code), cls)
    return out


def _raise_last() -> None:
    lib = _lib()
    code = int(lib.rfx_last_error_code())
    msg = (lib.rfx_last_error() or b"unknown failure").decode("utf-8", "replace")
    cls = _by_code().get(code, errors.ReflexError)
    raise cls(msg)


def _ids(values: Sequence[int]):
    return (c_uint32 * len(values))(*[int(v) for v in values])


def _ragged(lists: Sequence[Sequence[int]]):
    arrays = [_ids(l) for l in lists]
    ptrs = (POINTER(c_uint32) * len(lists))(*[ctypes.cast(a, POINTER(c_uint32)) for a in arrays])
    lens = (c_size_t * len(lists))(*[len(l) for l in lists])
    return arrays, ptrs, lens


class CModel:
    """A model handle of the C interface.  Not thread-safe, as the handle is not."""

    def __init__(self, handle: int):
        self._h = handle

    @classmethod
    def load(cls, model_dir: str, weights: Optional[str] = None, max_tokens: int = 0, max_batch: int = 0) -> "CModel":
        h = _lib().rfx_load(model_dir.encode(), weights.encode() if weights else None, max_tokens, max_batch)
        if not h:
            _raise_last()
        return cls(h)

    def close(self) -> None:
        if self._h:
            _lib().rfx_free(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 0.0, seed: int = -1,
                 stop_token_ids: Sequence[int] = ()) -> List[List[int]]:
        keep, ptrs, lens = _ragged(prompts)
        stops = _ids(stop_token_ids)
        samp = _Sampling(temperature, top_k, top_p, seed, ctypes.cast(stops, POINTER(c_uint32)), len(stop_token_ids))
        res = _GenerateResult()
        if _lib().rfx_generate(self._h, ptrs, lens, len(prompts), max_new_tokens, ctypes.byref(samp),
                               ctypes.byref(res)) != 0:
            _raise_last()
        try:
            return [[int(res.sequences[i].token_ids[j]) for j in range(res.sequences[i].num_tokens)]
                    for i in range(res.num_sequences)]
        finally:
            _lib().rfx_free_generate_result(ctypes.byref(res))

    def score(self, prompt: Sequence[int], candidates: Sequence[Sequence[int]],
              temperature: float = 1.0) -> Tuple[List[Tuple[float, float]], int, float]:
        """((score, probability) per candidate, best index, entropy in bits)."""
        p = _ids(prompt)
        keep, ptrs, lens = _ragged(candidates)
        res = _ScoreResult()
        if _lib().rfx_score(self._h, ctypes.cast(p, POINTER(c_uint32)), len(prompt), ptrs, lens, len(candidates),
                            temperature, ctypes.byref(res)) != 0:
            _raise_last()
        try:
            rows = [(float(res.candidates[i].score), float(res.candidates[i].probability))
                    for i in range(res.num_candidates)]
            return rows, int(res.best_idx), float(res.entropy)
        finally:
            _lib().rfx_free_score_result(ctypes.byref(res))

    def open_sequence(self) -> int:
        s = c_int64()
        if _lib().rfx_open_sequence(self._h, ctypes.byref(s)) != 0:
            _raise_last()
        return int(s.value)

    def close_sequence(self, sequence: int) -> None:
        if _lib().rfx_close_sequence(self._h, sequence) != 0:
            _raise_last()

    def step(self, entries: Sequence[Tuple[int, Sequence[int], Sequence[int]]]):
        """entries: (sequence, tokens, wanted places); float32 logits [wanted, vocab]
        as a NumPy array of its own (the library's buffer is freed before returning)."""
        import numpy as np

        keep = []
        arr = (_StepEntry * len(entries))()
        for i, (seq, toks, want) in enumerate(entries):
            t, w = _ids(toks), _ids(want)
            keep += [t, w]
            arr[i] = _StepEntry(seq, ctypes.cast(t, POINTER(c_uint32)), len(toks), ctypes.cast(w, POINTER(c_uint32)),
                                len(want))
        res = _StepResult()
        if _lib().rfx_step(self._h, arr, len(entries), ctypes.byref(res)) != 0:
            _raise_last()
        try:
            rows, V = int(res.rows), int(res.vocab)
            if rows == 0:
                return np.zeros((0, V), dtype=np.float32)
            return np.ctypeslib.as_array(res.logits, shape=(rows, V)).copy()
        finally:
            _lib().rfx_free_step_result(ctypes.byref(res))
