"""Rotary position encoding, half-split (NeoX) pairing.

For a head vector t[0..d) and i < rd/2:  theta = (float)pos / base^(2i/rd);
(t_i, t_{i+rd/2}) <- (t_i cos - t_{i+rd/2} sin, t_i sin + t_{i+rd/2} cos);
elements >= rd stay (src/kernels_cuda/rope.cu:9-37).  The part owns the table
of denominators base^(2i/rd), made once on the host in double precision and
rounded to 32-bit; the angle itself is computed per element in 32-bit inside
the fused kernel that the attention part launches.  Pairing and magnitude go
to that kernel as parameters (`Rotation`), so an encoding with consecutive
pairs or a scaled magnitude is another position part, not another kernel.
"""

from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

from ..config.spec import PositionSpec
from ..errors import InvalidInput
from .registry import Rotation, TensorInfo, register_position


@register_position("rope_neox")
class RotaryNeox:
    capturable = True

    def __init__(self, spec: PositionSpec, dtype: torch.dtype, device):
        if spec.rotary_dim % 2 or not (0 < spec.rotary_dim <= spec.head_dim):
            raise InvalidInput(
                f"rotary_dim must be even and in (0, head_dim], got {spec.rotary_dim}"
            )
        self.spec = spec
        half = spec.rotary_dim // 2
        # the C library's pow in double, element by element, then one rounding to 32-bit
        denom = [math.pow(float(spec.theta), 2.0 * i / float(spec.rotary_dim)) for i in range(half)]
        self.denominators = torch.tensor(denom, dtype=torch.float64).to(torch.float32).to(device)

    @classmethod
    def tensor_specs(cls, spec: PositionSpec) -> Dict[str, TensorInfo]:
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass

    def rotation(self) -> Rotation:
        return Rotation(self.denominators, self.spec.rotary_dim, "half", 1.0)
