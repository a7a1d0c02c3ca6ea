"""A causal language model put together from a `ModelSpec`.

embedding -> the layers in run order -> final norm -> head, with the logits
computed only at the rows a step asks for (the reference computes them for the
last row: src/model/dense.rs:2019-2025, src/model/mod.rs:1191-1202).  The model
holds parts and weights; what a step changes lives in the cache and the batch.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch

from .. import ops
from ..cache.specs import KVSpec, StateSpec
from ..config.spec import ModelSpec, RunEntry
from ..parts.registry import BLOCKS, NORMS, TensorInfo


@dataclass
class RunContext:
    """What a mixer gets besides its input rows."""

    batch: Any                 # StepBatch
    writes_cache: bool
    kv: Any = None             # KVView of this run's cache entry, if it has one
    state: Any = None          # [slots, *shape] tensor of this run's state, if any
    entry: int = -1


def expected_tensors(spec: ModelSpec) -> Dict[str, Tuple[Tuple[str, ...], TensorInfo]]:
    """tensor name -> (where it goes, TensorInfo) for the whole model."""
    out: Dict[str, Tuple[Tuple[str, ...], TensorInfo]] = {}
    out[spec.embedding_name] = (("embedding",), TensorInfo((spec.vocab_size, spec.hidden_size), "table"))
    for li, layer in enumerate(spec.layers):
        for name, (part, role, info) in BLOCKS.get(layer.block).tensor_names(layer).items():
            out[name] = (("layer", str(li), part, role), info)
    out[spec.final_norm_name] = (("final_norm",), TensorInfo((spec.final_norm.size,), "norm"))
    if not spec.tie_word_embeddings:
        out[spec.head_name] = (("head",), TensorInfo((spec.vocab_size, spec.hidden_size), "matrix"))
    return out


class CausalLM:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("dtype must be float32 or bfloat16")
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.layers = [BLOCKS.get(l.block)(l, dtype, self.device) for l in spec.layers]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, dtype, self.device)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None

    @property
    def capturable(self) -> bool:
        """True when every layer and the final norm declare `capturable = True`:
        their launches take positions, slots and lengths from device memory
        (`StepBatch`'s device fields) and nothing forces the host to wait, so a
        decode step can be captured once and replayed.  A part that walks host
        lists, or synchronises (a `.nonzero()`, an `.item()`), leaves the
        attribute out or sets it False, and the engine then runs every step
        eagerly."""
        return (all(bool(getattr(l, "capturable", False)) for l in self.layers)
                and bool(getattr(self.final_norm, "capturable", False)))

    # --- weights ----------------------------------------------------------
    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """`tensors`: every name of `expected_tensors`, already checked."""
        exp = expected_tensors(self.spec)
        per_layer: Dict[int, Dict[str, Dict[str, torch.Tensor]]] = {}
        for name, (where, _info) in exp.items():
            t = tensors[name]
            if where[0] == "embedding":
                self.embedding = t.to(device=self.device, dtype=self.dtype).contiguous()
            elif where[0] == "head":
                self.head = t.to(device=self.device, dtype=self.dtype).contiguous()
            elif where[0] == "final_norm":
                self.final_norm.bind({"weight": t})
            else:
                _, li, part, role = where
                per_layer.setdefault(int(li), {}).setdefault(part, {})[role] = t
        for li, layer in enumerate(self.layers):
            layer.bind(per_layer.get(li, {}))
        if self.spec.tie_word_embeddings:
            self.head = self.embedding  # the same storage, no copy

    # --- cache ------------------------------------------------------------
    def cache_entry_specs(self) -> Dict[int, Any]:
        out = {}
        for entry, li in self.spec.cache_entries().items():
            mixer = self.layers[li].mixer
            out[entry] = mixer.cache_spec() if hasattr(mixer, "cache_spec") else None
        return out

    # --- forward ----------------------------------------------------------
    def hidden_states(self, batch, cache) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        ops.prof_mark("start")
        # a token id outside the vocabulary (possible only for ids fed from the device)
        # gives a zero row and sets the device's error word, which `check_errors` reads
        h = ops.embed(self.embedding, batch.tokens, self.spec.embedding_scale,
                      ops.device_error_word(self.device))
        ops.prof_mark("embed")
        pending = None
        order = self.spec.run_order
        for i, run in enumerate(order):
            # the norm that will consume this run's result: the next run's first norm, or the final one
            next_norm = (getattr(self.layers[order[i + 1].layer], "fusable_first_norm", None)
                         if i + 1 < len(order) else self.final_norm)
            ops.workspace.next_phase()  # this run's working memory; the last run's results stay readable
            ctx = RunContext(batch=batch, writes_cache=run.writes_cache, entry=run.cache)
            kind = cache.has(run.cache)
            if kind == "kv":
                ctx.kv = cache.kv(run.cache)
            elif kind == "state":
                ctx.state = cache.state(run.cache)
            layer = self.layers[run.layer]
            if hasattr(layer, "fusable_first_norm"):
                h, pending = layer.forward(h, pending, ctx, next_norm=next_norm)
            else:
                h, pending = layer.forward(h, pending, ctx)
        return h, pending

    def logits(self, hidden: torch.Tensor, pending, rows: torch.Tensor, rows_host=None) -> torch.Tensor:
        """Final norm and head on the wanted rows only; float32 [len(rows), V]."""
        if isinstance(pending, ops.NormedInput):
            # fused decode path: hidden already holds the last delta
            if rows_host is not None and list(rows_host) == list(range(hidden.shape[0])):
                normed = pending  # every row wanted, in order: the head product takes them as they are
            else:
                normed = self.final_norm(hidden, rows=rows)
        else:
            normed = self.final_norm(hidden, delta=pending, rows=rows)
        out = ops.linear(normed, self.head, out_dtype=torch.float32, own=True)  # the caller's to keep
        if self.spec.logit_scale != 1.0:
            out = out * self.spec.logit_scale
        ops.prof_mark("head")
        return out

    def normed_rows(self, hidden: torch.Tensor, pending, rows: torch.Tensor) -> torch.Tensor:
        """The final norm on the wanted rows, in the model's dtype."""
        if isinstance(pending, ops.NormedInput):
            return self.final_norm(hidden, rows=rows)  # hidden already holds the last delta
        return self.final_norm(hidden, delta=pending, rows=rows)

    def scores(self, batch, cache, ids: torch.Tensor) -> torch.Tensor:
        """For each wanted row the head's logit of one given token id
        (`ids`, int32 on the device, one per wanted row), float32 [wanted]: only
        those rows of the head are read (src/model/dense.rs:2073-2133)."""
        h, pending = self.hidden_states(batch, cache)
        out = ops.gather_dot(self.normed_rows(h, pending, batch.want_rows), self.head, ids)
        if self.spec.logit_scale != 1.0:
            out = out * self.spec.logit_scale
        ops.prof_mark("head")
        return out

    def forward(self, batch, cache) -> torch.Tensor:
        h, pending = self.hidden_states(batch, cache)
        return self.logits(h, pending, batch.want_rows, batch.want_rows_host)
