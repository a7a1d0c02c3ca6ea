"""Rotary position encoding, half-split (NeoX) pairing.

For a head vector t[0..d) and i < rd/2:  theta = (float)pos / base^(2i/rd);
(t_i, t_{i+rd/2}) <- (t_i cos - t_{i+rd/2} sin, t_i sin + t_{i+rd/2} cos);
elements >= rd stay (src/kernels_cuda/rope.cu:9-37).  The part owns the table
of denominators base^(2i/rd), made once on the host in double precision and
rounded to 32-bit; the angle itself is computed per element in 32-bit inside
the fused kernel that the attention part launches.
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..config.spec import PositionSpec
from ..errors import InvalidInput
from .registry import TensorInfo, register_position


@register_position("rope_neox")
class RotaryNeox:
    def __init__(self, spec: PositionSpec, dtype: torch.dtype, device):
        if spec.rotary_dim % 2 or not (0 < spec.rotary_dim <= spec.head_dim):
            raise InvalidInput(
                f"rotary_dim must be even and in (0, head_dim], got {spec.rotary_dim}"
            )
        self.spec = spec
        half = spec.rotary_dim // 2
        exponents = torch.arange(half, dtype=torch.float64) * 2.0 / float(spec.rotary_dim)
        denom = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), exponents)
        self.denominators = denom.to(torch.float32).to(device)

    @classmethod
    def tensor_specs(cls, spec: PositionSpec) -> Dict[str, TensorInfo]:
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass

    def rotation(self) -> Tuple[Optional[torch.Tensor], int]:
        return self.denominators, self.spec.rotary_dim
