"""RMSNorm over the last dimension, statistics in 32-bit.

y = (x * r) * (weight_offset + w),  r = 1 / sqrt(mean(x^2) + eps)
(src/kernels_cuda/rmsnorm.cuh:14-40, src/kernels_cuda/rmsnorm.cu:44-52).  The
residual add that precedes a norm is fused into it, as the reference's decode
path does (src/kernels_cuda/decode_ops.cu:10-35).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..config.spec import NormSpec
from .registry import TensorInfo, register_norm


@register_norm("rmsnorm")
class RMSNorm:
    capturable = True  # launches read nothing from the host: may be captured into a CUDA graph

    def __init__(self, spec: NormSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def tensor_specs(cls, spec: NormSpec) -> Dict[str, TensorInfo]:
        return {"weight": TensorInfo((spec.size,), "norm")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].to(device=self.device, dtype=torch.float32).contiguous()

    def __call__(self, residual: torch.Tensor, delta: Optional[torch.Tensor] = None,
                 rows: Optional[torch.Tensor] = None, update: bool = True) -> torch.Tensor:
        return ops.rmsnorm(residual, self.weight, self.spec.eps, self.dtype, delta=delta,
                           update_residual=update, rows=rows,
                           weight_offset=self.spec.weight_offset)
