"""Sampling options, with the reference's names and meanings
(src/sampling.rs:41-66): `temperature <= 0` (the default) or NaN is greedy
argmax with no random draw; a positive temperature samples from the softmax,
after `top_k` (keep the k most probable) and then `top_p` (keep the shortest
most-probable prefix whose probability reaches top_p); `seed` makes the draws
reproducible; `stop_token_ids` end a generation (the stop token is kept).
"""

from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import Optional, Tuple

from ..errors import InvalidInput


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    seed: Optional[int] = None
    stop_token_ids: Tuple[int, ...] = ()

    def is_greedy(self) -> bool:
        return math.isnan(self.temperature) or self.temperature <= 0.0

    def validate(self) -> None:
        """The reference's checks (src/sampling.rs:215-239)."""
        if self.is_greedy():
            return
        if not math.isfinite(self.temperature):
            raise InvalidInput(
                f"sample: temperature must be positive and finite when sampling, got {self.temperature}")
        if self.top_k is not None and self.top_k < 1:
            raise InvalidInput("sample: top_k must be at least 1")
        if self.top_p is not None and not (math.isfinite(self.top_p) and 0.0 <= self.top_p <= 1.0):
            raise InvalidInput(f"sample: top_p must be in [0, 1], got {self.top_p}")


_MASK = (1 << 64) - 1


def _mix(x: int) -> int:
    """splitmix64's finaliser."""
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform(seed: int, request: int, step: int) -> float:
    """A uniform number in [0, 1) that depends only on (seed, request, step), so
    a request's draws do not depend on what else is in its batch.  (The
    reference seeds one ChaCha generator per call, src/sampling.rs:72-77, which
    cannot be reproduced outside its Rust crate.)"""
    x = _mix(_mix(_mix(seed & _MASK) ^ (request & _MASK)) ^ (step & _MASK))
    return (x >> 40) / float(1 << 24)


def fresh_seed() -> int:
    return int.from_bytes(os.urandom(8), "little")
