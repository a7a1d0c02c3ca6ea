"""Block arrangements: how a layer's parts are wired around the residual.

"prenorm": h += mixer(norm1(h)); h += ffn(norm2(h))
(src/model/dense.rs:1441-1484).  The residual stream is 32-bit; each add is
fused into the norm that follows it, so a block hands its last delta on as
`pending` and the next block's (or the model's final) norm adds it
(src/model/decode_step.rs:199-210, 293-300).
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..config.spec import LayerSpec, names_dict
from .registry import FEED_FORWARDS, MIXERS, NORMS, TensorInfo, register_block


@register_block("prenorm")
class PreNormBlock:
    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm, dtype, device)
        self.feed_forward_norm = NORMS.get(spec.feed_forward_norm.kind)(
            spec.feed_forward_norm, dtype, device)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, dtype, device)
        self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, dtype, device)

    @property
    def fusable_first_norm(self):
        """The norm this layer starts with, if the product before it may begin it
        (the mixer then gets rows that await their norm factor, an
        `ops.NormedInput`, which only a mixer that says so accepts); else None."""
        return self.mixer_norm if getattr(self.mixer, "accepts_normed_input", False) else None

    @property
    def capturable(self) -> bool:
        """Whether every part of the layer allows its launches to be captured."""
        return all(bool(getattr(p, "capturable", False))
                   for p in (self.mixer_norm, self.feed_forward_norm, self.mixer, self.feed_forward))

    @classmethod
    def tensor_names(cls, spec: LayerSpec) -> Dict[str, Tuple[str, str, TensorInfo]]:
        """full tensor name -> (part, role, info) for every tensor of the layer."""
        out: Dict[str, Tuple[str, str, TensorInfo]] = {}
        block_names = names_dict(spec.names)

        def add(part: str, infos: Dict[str, TensorInfo], names: Dict[str, str]) -> None:
            for role, info in infos.items():
                suffix = names.get(role, role)
                out[spec.prefix + suffix] = (part, role, info)

        add("mixer_norm", {"weight": NORMS.get(spec.mixer_norm.kind).tensor_specs(spec.mixer_norm)["weight"]},
            {"weight": block_names.get("mixer_norm", "mixer_norm.weight")})
        add("feed_forward_norm",
            {"weight": NORMS.get(spec.feed_forward_norm.kind).tensor_specs(spec.feed_forward_norm)["weight"]},
            {"weight": block_names.get("feed_forward_norm", "feed_forward_norm.weight")})
        add("mixer", MIXERS.get(spec.mixer.kind).tensor_specs(spec.mixer), names_dict(spec.mixer.names))
        add("feed_forward", FEED_FORWARDS.get(spec.feed_forward.kind).tensor_specs(spec.feed_forward),
            names_dict(spec.feed_forward.names))
        return out

    def bind(self, by_part: Dict[str, Dict[str, torch.Tensor]]) -> None:
        self.mixer_norm.bind(by_part.get("mixer_norm", {}))
        self.feed_forward_norm.bind(by_part.get("feed_forward_norm", {}))
        self.mixer.bind(by_part.get("mixer", {}))
        self.feed_forward.bind(by_part.get("feed_forward", {}))

    def forward(self, hidden: torch.Tensor, pending, ctx, next_norm=None):
        """`pending` is what the block before left: a delta still to be added to
        `hidden`, None (nothing to add), or an `ops.NormedInput`: `hidden` already
        holds the sum and the rows only await this block's first norm factor.
        `next_norm` is the norm that will consume this block's result; parts that
        can fuse the residual add and that norm into their last product do so."""
        from .. import ops

        if isinstance(pending, ops.NormedInput):
            x = pending
        else:
            x = self.mixer_norm(hidden, delta=pending)
            ops.prof_mark("norm")
        if getattr(self.mixer, "supports_fused_residual", False):
            ffn_norm = self.feed_forward_norm if getattr(self.feed_forward, "accepts_normed_input", False) else None
            a = self.mixer.forward(x, ctx, residual=(hidden, ffn_norm))
        else:
            a = self.mixer.forward(x, ctx)
        if isinstance(a, ops.NormedInput):
            x = a
        else:
            x = self.feed_forward_norm(hidden, delta=a)
            ops.prof_mark("norm")
        if getattr(self.feed_forward, "supports_fused_residual", False):
            f = self.feed_forward.forward(x, residual=(hidden, next_norm))
        else:
            f = self.feed_forward.forward(x)
        return hidden, f
