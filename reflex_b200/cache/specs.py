"""What a mixer asks of the cache."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class KVSpec:
    """Keys and values per position: `n_kv_heads` vectors of `head_dim` each.
    With a `window` only the last `window` positions are ever read again, so
    the store gives older pages back."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    # size of a value vector when it differs from a key vector's (a compressed
    # latent cache; the reference's attention parameters carry separate K and V
    # strides for it, src/kernels_cuda/attention_online.cu:22-23); None: head_dim
    v_head_dim: Optional[int] = None

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim


@dataclass(frozen=True)
class StateSpec:
    """Per-sequence state of fixed size (recurrent and convolutional mixers):
    not indexed by position, zero at a sequence's start, updated in place by
    each step (the reference's examples: src/model/hybrid.rs:131-140,
    src/model/granite_hybrid.rs:67-74)."""

    shape: Tuple[int, ...]
    dtype: str = "float32"
