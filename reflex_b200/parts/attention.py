"""Grouped-query attention over the paged cache.

q = x Wq^T, k = x Wk^T, v = x Wv^T (no bias); per-head RMSNorm of q and k when
the spec has one; rotary encoding of q and k; k and v written to the cache at
the row's position; then for the query at position p, head h (kv head
h / group): keys j with 0 <= p - j < window (all j <= p without a window),
softmax((q . k_j) * scale) in 32-bit, weighted sum of v_j; out = attn Wo^T
(src/model/dense.rs:1337-1431; src/kernels_cuda/attention_online.cuh:64-102).
The q, k, v weights are stacked into one matrix at load; the reference fuses
the three products by kernel instead (src/kernels_cuda/gemv_fused.cu:16-87).

The part knows sizes only from its spec.  What it needs from the step is in
`ctx`: row positions, row slots, and the cache entry's pages and page table.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..cache.specs import KVSpec
from ..config.spec import MixerSpec
from ..errors import InvalidInput
from .registry import NORMS, POSITIONS, TensorInfo, register_mixer


@register_mixer("gqa_attention")
class GQAttention:
    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device):
        if spec.num_heads % spec.num_kv_heads:
            raise InvalidInput("num_heads must be a multiple of num_kv_heads")
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.position = (
            POSITIONS.get(spec.position.kind)(spec.position, dtype, device)
            if spec.position is not None
            else None
        )
        self.qkv = None
        self.q_only = None
        self.o = None
        self.q_norm = None
        self.k_norm = None

    @classmethod
    def tensor_specs(cls, spec: MixerSpec) -> Dict[str, TensorInfo]:
        H, d = spec.hidden_size, spec.head_dim
        out = {
            "q_proj": TensorInfo((spec.num_heads * d, H), "matrix"),
            "k_proj": TensorInfo((spec.num_kv_heads * d, H), "matrix"),
            "v_proj": TensorInfo((spec.num_kv_heads * d, H), "matrix"),
            "o_proj": TensorInfo((H, spec.num_heads * d), "matrix"),
        }
        if spec.qk_norm is not None:
            out["q_norm"] = TensorInfo((d,), "norm")
            out["k_norm"] = TensorInfo((d,), "norm")
        return out

    def cache_spec(self) -> KVSpec:
        return KVSpec(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        def dev(t):
            return t.to(device=self.device, dtype=self.dtype)

        q = dev(tensors["q_proj"])
        self.qkv = torch.cat([q, dev(tensors["k_proj"]), dev(tensors["v_proj"])], dim=0).contiguous()
        # rows [0, nq*d) of the stacked matrix: the query part, for runs that
        # read another run's keys and values
        self.q_only = self.qkv[: q.shape[0]]
        self.o = dev(tensors["o_proj"]).contiguous()
        if self.spec.qk_norm is not None:
            self.q_norm = tensors["q_norm"].to(device=self.device, dtype=torch.float32).contiguous()
            self.k_norm = tensors["k_norm"].to(device=self.device, dtype=torch.float32).contiguous()

    supports_fused_residual = True
    accepts_normed_input = True  # its first product finishes a norm that the product before began

    @property
    def capturable(self) -> bool:
        """Positions, slots and the page table are read from device memory, so a
        decode step's launches may be captured, if the position part's may."""
        return self.position is None or bool(getattr(self.position, "capturable", False))

    def forward(self, x, ctx, residual=None):
        """x: normed rows (or rows awaiting their norm factor, `ops.NormedInput`).
        With `residual` = (hidden, next norm) the output projection may add
        itself to `hidden`; it then returns the rows for the product after that
        norm (an `ops.NormedInput`) or None (added, the norm not begun).
        Otherwise the delta [rows, hidden] is returned."""
        s = self.spec
        kv = ctx.kv  # the cache entry's view
        batch = ctx.batch
        w = self.qkv if ctx.writes_cache else self.q_only
        rotation = None if self.position is None else self.position.rotation()
        norm = s.qk_norm
        if ops.qkv_fused_takes(x, s.head_dim, rotation, w):
            # a few rows: norms, rotation and the cache write are the product's epilogue
            q = ops.qkv_fused(
                x, w, self.q_norm, self.k_norm, norm.eps if norm else 0.0,
                norm.weight_offset if norm else 0.0, rotation, batch.row_pos, batch.row_slot,
                kv.k_pages, kv.v_pages, kv.page_table, kv.page_size, s.num_heads, s.num_kv_heads,
                s.head_dim, ctx.writes_cache)
            ops.prof_mark("qkv_gemm")
        else:
            qkv = ops.linear(x, w, out_dtype=torch.float32 if x.shape[0] <= ops.GEMV_MAX_ROWS else None)
            ops.prof_mark("qkv_gemm")
            q = ops.qkv_post(
                qkv, self.q_norm, self.k_norm, norm.eps if norm else 0.0,
                norm.weight_offset if norm else 0.0, rotation, batch.row_pos, batch.row_slot,
                kv.k_pages, kv.v_pages, kv.page_table, kv.page_size, s.num_heads, s.num_kv_heads,
                s.head_dim, ctx.writes_cache, self.dtype)
            ops.prof_mark("norm_rope")
        attn = ops.attention(q, kv.k_pages, kv.v_pages, kv.page_table, kv.page_size, batch,
                             s.num_heads, s.num_kv_heads, s.head_dim, s.window, s.scale)
        ops.prof_mark("attn")
        if residual is not None:
            fused = ops.linear_residual(attn, self.o, residual[0], residual[1])
            if fused is not None:
                ops.prof_mark("o_proj")
                return None if fused is ops.ADDED else fused  # None: nothing left to add
        out = ops.linear(attn, self.o, out_dtype=torch.float32)
        ops.prof_mark("o_proj")
        return out
