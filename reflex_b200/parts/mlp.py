"""Gated feed-forward (SwiGLU), dense.

gate = x Wg^T, up = x Wu^T, act = gate / (1 + exp(-gate)) * up, out = act Wd^T
(src/model/dense.rs:1476-1481, src/kernels_cuda/silu_and_mul.cu:7-23).  The
gate and up weights are woven into one [2I, H] matrix at load, row 2j = gate_j
and row 2j + 1 = up_j, so that one product serves both (the reference's decode
path fuses them by kernel, src/kernels_cuda/gemv_fused.cu:143-203) and the
activation can be that product's epilogue; reordering rows changes no output.
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.spec import FeedForwardSpec
from .registry import TensorInfo, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU:
    capturable = True  # launches read nothing from the host: may be captured into a CUDA graph

    def __init__(self, spec: FeedForwardSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.gate_up = None
        self.down = None

    @classmethod
    def tensor_specs(cls, spec: FeedForwardSpec) -> Dict[str, TensorInfo]:
        H, I = spec.hidden_size, spec.intermediate_size
        return {
            "gate_proj": TensorInfo((I, H), "matrix"),
            "up_proj": TensorInfo((I, H), "matrix"),
            "down_proj": TensorInfo((H, I), "matrix"),
        }

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        def dev(t):
            return t.to(device=self.device, dtype=self.dtype)

        g, u = dev(tensors["gate_proj"]), dev(tensors["up_proj"])
        self.gate_up = torch.stack([g, u], dim=1).reshape(2 * g.shape[0], g.shape[1]).contiguous()
        self.down = dev(tensors["down_proj"]).contiguous()

    supports_fused_residual = True
    accepts_normed_input = True  # its first product finishes a norm that the product before began

    def forward(self, x, residual=None):
        """With `residual` = (hidden, next norm) the down projection may add itself
        to `hidden`; it then returns the rows for the product after that norm
        (`ops.NormedInput`) or None (added, the norm not begun).  Otherwise it
        returns the delta."""
        act = ops.linear_swiglu(x, self.gate_up)
        ops.prof_mark("ffn_gate_up")
        if residual is not None:
            fused = ops.linear_residual(act, self.down, residual[0], residual[1])
            if fused is not None:
                ops.prof_mark("ffn_down")
                return None if fused is ops.ADDED else fused  # None: nothing left to add
        out = ops.linear(act, self.down, out_dtype=torch.float32)
        ops.prof_mark("ffn_down")
        return out
