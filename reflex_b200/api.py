"""The Python entry point, in the manner of the reference's `Model`
(src/model/mod.rs:781-829 load, :1003-1022 generate, :1123-1132
system1_evaluate, :933-972 forward_prompt) and of its C interface
(include/reflex_engine.h:185-328): load a model once, then generate or score
with it.  The reference takes text and owns a tokenizer; this library works on
token ids.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Union

import torch

from .engine.generate import GenerationStats, generate as _generate
from .engine.step import Engine
from .errors import InvalidInput
from .sampling import Sampler, SamplingParams

_DTYPES = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "f32": torch.float32,
           "float32": torch.float32, "fp32": torch.float32}


def resolve_weights(flag: Optional[str] = None, default: str = "bf16") -> str:
    """The weights option: `flag` if given, else the environment's
    `REFLEX_WEIGHTS` if set and not empty, else `default`
    (src/model/loading.rs:44-62; `check` passes "f32" as its default)."""
    import os

    if flag is not None:
        if flag not in _DTYPES:
            raise InvalidInput(f"weights must be one of {sorted(_DTYPES)}, got {flag!r}")
        return flag
    env = os.environ.get("REFLEX_WEIGHTS", "")
    if env:
        if env not in _DTYPES:
            raise InvalidInput(f"REFLEX_WEIGHTS: weights must be one of {sorted(_DTYPES)}, got {env!r}")
        return env
    return default


@dataclass
class EngineOptions:
    """What is fixed when a model is loaded (the reference's `LoadOptions`,
    src/model/loading.rs:91-98, and its environment switches read once at load).
    `weights` None: `REFLEX_WEIGHTS`, else bfloat16.  The cache's element type
    follows the weights' (32-bit with "f32").  `max_tokens` sizes the cache
    (tokens held by all live sequences, each rounded up to a page);
    `max_batch` is the most sequences the generation loop runs together."""

    weights: Optional[str] = None
    device: str = "cuda:0"
    max_tokens: int = 16384
    max_batch: int = 64
    use_graphs: bool = True


@dataclass
class System1CandidateResult:
    token_ids: List[int]
    score: float  # sum of the raw head logits of the candidate's tokens


@dataclass
class System1Response:
    results: List[System1CandidateResult]
    probabilities: List[float]
    entropy: float  # bits

    @property
    def best_idx(self) -> int:
        return max(range(len(self.probabilities)), key=lambda i: (self.probabilities[i], i))


def softmax_scores_with_temperature(scores: Sequence[float], temperature: float) -> List[float]:
    """src/calibration.rs:21-47."""
    if len(scores) == 0:
        raise InvalidInput("softmax_scores: scores must not be empty")
    if not math.isfinite(temperature) or temperature <= 0.0:
        raise InvalidInput(f"softmax_scores: temperature must be positive and finite, got {temperature}")
    scaled = [s / temperature for s in scores]
    m = max(scaled)
    exps = [math.exp(s - m) for s in scaled]
    total = sum(exps)
    if not math.isfinite(total) or total <= 0.0:
        raise InvalidInput(f"softmax_scores: softmax sum is non-finite or non-positive ({total})")
    return [e / total for e in exps]


def shannon_entropy(probabilities: Sequence[float]) -> float:
    """Base-2 entropy, 0 log 0 = 0 (src/calibration.rs:59-74)."""
    if len(probabilities) == 0:
        raise InvalidInput("shannon_entropy: probabilities must not be empty")
    if any(not math.isfinite(p) for p in probabilities):
        raise InvalidInput("shannon_entropy: probabilities must all be finite")
    return -sum(0.0 if p <= 0.0 else p * math.log2(p) for p in probabilities)


class Model:
    """A loaded model with its cache and step function."""

    def __init__(self, causal_lm, max_tokens: int = 16384, max_batch: int = 64, use_graphs: bool = True):
        self.lm = causal_lm
        self.spec = causal_lm.spec
        self.max_batch = max_batch
        self.engine = Engine(causal_lm, max_tokens=max_tokens, use_graphs=use_graphs)
        self.last_stats: Optional[GenerationStats] = None
        # the generation loop keeps the device one step ahead of the host
        self.decode_ahead = True

    @classmethod
    def load(cls, model_dir: str, weights: Optional[str] = None, device: Optional[str] = None,
             options: Optional[EngineOptions] = None, **kw) -> "Model":
        """`weights`: "bf16" (serving precision) or "f32" (everything in true
        32-bit), the role of the reference's `--weights f16|f32`
        (src/model/loading.rs:44-62); None: `REFLEX_WEIGHTS`, else bfloat16.
        `options` gives the same and the cache's size as one object; arguments
        given beside it win."""
        from .weights.loader import load_model

        o = options or EngineOptions()
        weights = resolve_weights(weights if weights is not None else o.weights)
        device = device if device is not None else o.device
        sizes = {"max_tokens": o.max_tokens, "max_batch": o.max_batch, "use_graphs": o.use_graphs}
        unknown = set(kw) - set(sizes)
        if unknown:
            raise InvalidInput(f"unknown load options: {sorted(unknown)}")
        sizes.update(kw)
        return cls(load_model(model_dir, _DTYPES[weights], device), **sizes)

    @property
    def weights_dtype(self) -> str:
        return "bf16" if self.lm.dtype == torch.bfloat16 else "f32"

    # ------------------------------------------------------------------
    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]], max_new_tokens: int,
                 sampling: Optional[SamplingParams] = None,
                 on_token: Optional[Callable[[int, int], None]] = None):
        """Greedy by default.  One prompt (a list of ids) gives a list of ids;
        a list of prompts gives a list of lists.  Stop tokens are the model's
        end-of-sequence ids and `sampling.stop_token_ids`; the stop token is
        kept in the output."""
        sampling = sampling or SamplingParams()
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        plist = [list(prompts)] if single else [list(p) for p in prompts]
        sampler = Sampler(sampling, self.lm.device)
        stops = tuple(self.spec.eos_token_ids) + tuple(sampling.stop_token_ids)
        stats = GenerationStats()
        out = _generate(self.engine, plist, max_new_tokens, sampler.pick, stops,
                        max_batch=self.max_batch, on_token=on_token, stats=stats,
                        pick_async=sampler.pick_async if self.decode_ahead else None)
        self.last_stats = stats
        return out[0] if single else out

    def forward_prompt(self, prompt: Sequence[int]) -> torch.Tensor:
        """Float32 logits [len(prompt), vocab] of one whole prompt."""
        s = self.engine.open()
        try:
            logits = self.engine.step([(s, list(prompt), list(range(len(prompt))))]).clone()
            self.engine.check_errors()
            return logits
        finally:
            self.engine.close(s)

    def system1_evaluate(self, prompt: Sequence[int], candidates: Sequence[Sequence[int]],
                         temperature: float = 1.0) -> System1Response:
        """Score continuations of a prompt in one prefill step.  A candidate's
        score is the sum of the raw head logits of its tokens, each read at the
        row before it with the candidate's earlier tokens teacher-forced
        (src/model/dense.rs:2073-2133, src/model/mod.rs:405-413); probabilities
        are the softmax of the scores over `temperature`, entropy in bits
        (src/model/mod.rs:1140-1164).  All candidates run as sequences of one
        batch."""
        if len(candidates) == 0:
            raise InvalidInput("system1 needs at least one candidate")
        if len(prompt) == 0:
            raise InvalidInput("prompt is empty")
        V = self.spec.vocab_size
        for ci, c in enumerate(candidates):
            if len(c) == 0:
                raise InvalidInput("a candidate has no tokens")
            for t in c:  # every id, the last one too: it indexes the head, it is never embedded
                if not (0 <= int(t) < V):
                    raise InvalidInput(f"candidate {ci}: token id {t} is outside the vocabulary [0, {V})")
        eng = self.engine
        if len(candidates) > eng.cache.slots.free_count:
            from .errors import OutOfMemory

            raise OutOfMemory(f"system1 needs a cache slot per candidate: {len(candidates)} candidates, "
                              f"{eng.cache.slots.free_count} slots free")
        seqs: List[int] = []
        try:
            for _ in candidates:
                seqs.append(eng.open())
            P = len(prompt)
            entries = []
            for s, c in zip(seqs, candidates):
                toks = list(prompt) + list(c[:-1])
                entries.append((s, toks, list(range(P - 1, P - 1 + len(c))), list(c)))
            # the head's rows of the candidates' tokens only, not the whole vocabulary
            picked = eng.step_scores(entries).tolist()
            eng.check_errors()
        finally:
            for s in seqs:
                eng.close(s)
        results, r = [], 0
        for c in candidates:
            results.append(System1CandidateResult(list(c), float(sum(picked[r:r + len(c)]))))
            r += len(c)
        probs = softmax_scores_with_temperature([x.score for x in results], temperature)
        return System1Response(results, probs, shannon_entropy(probs))
