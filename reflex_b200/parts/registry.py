"""Registries of the parts a layer is put together from.

A part is registered under the `kind` its spec names.  Nothing else in the
framework refers to a part's class, so a new mixer, feed-forward, norm,
position encoding or block arrangement is one decorated class, in the
framework or outside it (a test can register a toy mixer).

Interfaces (duck-typed; `spec` is the part's record from `config.spec`):

  every part
    tensor_specs(spec) -> {role: TensorInfo}     classmethod; what it loads
    __init__(spec, dtype, device)
    bind(tensors: {role: Tensor})                takes ownership of its weights
    capturable = True                            optional: its launches take everything that
                                                 changes from step to step out of device memory
                                                 and never wait for the host, so a decode step
                                                 may be captured into a CUDA graph; absent or
                                                 False: the engine runs every step eagerly

  norm            __call__(residual_f32, delta=None, rows=None, update=True) -> normed
  position        rotation() -> Rotation (below) | None
  mixer           cache_spec() -> KVSpec | StateSpec | None
                  forward(x, ctx) -> delta [rows, hidden]
  feed-forward    forward(x) -> delta [rows, hidden]
  block           forward(hidden_f32, pending_delta, ctx) -> (hidden_f32, pending_delta)
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Tuple

from ..errors import UnsupportedArchitecture


@dataclass(frozen=True)
class TensorInfo:
    shape: Tuple[int, ...]
    # "matrix": a linear layer's weight, kept in the compute dtype, drawn N(0, 0.02)
    # "table":  an embedding table, same
    # "norm":   a norm's weight, kept 32-bit, drawn 1 + U(-0.1, 0.1)
    role: str
    optional: bool = False


@dataclass(frozen=True)
class Rotation:
    """What a rotary position encoding hands to the mixer that applies it.

    A head vector's first `rotary_dim` elements are rotated in pairs; pair i
    turns by the angle position / denominators[i] (32-bit division), and the
    cosine and sine are multiplied by `magnitude` (1.0: a pure rotation; a
    frequency-scaled encoding's attention factor otherwise,
    src/model/kernels.rs:3086-3129).  `pairing` says which elements form pair i:
    "half" (i, i + rotary_dim / 2) or "consecutive" (2i, 2i + 1)
    (src/model/config.rs:15-28).  Variants that differ in their frequencies
    differ only in the table."""

    denominators: "object"  # float32 tensor [rotary_dim / 2] on the device
    rotary_dim: int
    pairing: str = "half"
    magnitude: float = 1.0


PAIRINGS = {"half": 0, "consecutive": 1}


class _Registry:
    def __init__(self, what: str):
        self.what = what
        self._items: Dict[str, type] = {}

    def register(self, kind: str) -> Callable[[type], type]:
        def deco(cls: type) -> type:
            self._items[kind] = cls
            return cls

        return deco

    def get(self, kind: str) -> type:
        try:
            return self._items[kind]
        except KeyError:
            raise UnsupportedArchitecture(
                f"no {self.what} registered under {kind!r}; known: {sorted(self._items)}"
            ) from None

    def kinds(self):
        return sorted(self._items)


MIXERS = _Registry("mixer")
FEED_FORWARDS = _Registry("feed-forward")
NORMS = _Registry("norm")
POSITIONS = _Registry("position encoding")
BLOCKS = _Registry("block arrangement")

register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_norm = NORMS.register
register_position = POSITIONS.register
register_block = BLOCKS.register
