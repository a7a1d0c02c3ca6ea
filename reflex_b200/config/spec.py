"""Architecture-neutral description of a model as data.

A model is a list of layers; a layer is a block arrangement of a mixer, a
feed-forward and its norms; the order in which layers run is a list of its own.
Every size and constant lives in these records, none in the parts' code, and a
part never learns which architecture it belongs to.  An architecture module
(e.g. `reflex_b200.models.qwen3`) turns its typed config.json record into a
`ModelSpec`; everything below that (weights, cache, step) works from the
`ModelSpec` alone.

Each `*Spec` names its part by `kind`, the key under which the part's class is
registered (`reflex_b200.parts.registry`).  `names` maps the part's local
tensor roles to the checkpoint's tensor-name suffixes, so a rename in a
checkpoint format is one line in the architecture module.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last dimension of `size` elements."""

    kind: str  # "rmsnorm"
    size: int
    eps: float
    # y = x * r * (weight_offset + w); 0.0 is the reference's plain weight
    # (src/kernels_cuda/rmsnorm.cu:44-52), 1.0 the "1 + w" variant.
    weight_offset: float = 0.0


@dataclass(frozen=True)
class PositionSpec:
    """A position encoding applied to query and key head vectors."""

    kind: str  # "rope_neox"
    head_dim: int
    rotary_dim: int
    theta: float
    params: Tuple[Tuple[str, Any], ...] = ()


@dataclass(frozen=True)
class MixerSpec:
    """The sequence-mixing half of a layer.  For attention: sizes of the heads,
    the optional per-head q/k norm, the position encoding and the window."""

    kind: str  # "gqa_attention"
    hidden_size: int
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 0.0
    # query i sees key j iff 0 <= i - j < window (src/model/config.rs:1184-1185);
    # None = every earlier key.
    window: Optional[int] = None
    qk_norm: Optional[NormSpec] = None
    position: Optional[PositionSpec] = None
    names: Tuple[Tuple[str, str], ...] = ()
    params: Tuple[Tuple[str, Any], ...] = ()


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str  # "swiglu"
    hidden_size: int
    intermediate_size: int
    names: Tuple[Tuple[str, str], ...] = ()
    params: Tuple[Tuple[str, Any], ...] = ()


@dataclass(frozen=True)
class LayerSpec:
    """One layer: which block arrangement, and the parts it arranges.

    `prefix` is prepended to every tensor name of the layer's parts."""

    block: str  # "prenorm"
    prefix: str
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    mixer_norm: NormSpec
    feed_forward_norm: NormSpec
    names: Tuple[Tuple[str, str], ...] = ()
    # further norms of the arrangement, by role (sandwich norms after the mixer and
    # after the feed-forward, before the residual add: src/model/dense.rs:72-83,
    # 928-930), and any other option of it: a block registered outside the
    # framework reads them, the framework only carries them
    extra_norms: Tuple[Tuple[str, NormSpec], ...] = ()
    params: Tuple[Tuple[str, Any], ...] = ()


@dataclass(frozen=True)
class RunEntry:
    """One position of the run order.

    `layer` indexes `ModelSpec.layers` (a layer may appear more than once: its
    weights are then shared).  `cache` names the cache entry this run uses; by
    default every run has an entry of its own.  With `writes_cache=False` the
    run reads the entry that an earlier run filled (key/value sharing between
    layers) and stores nothing."""

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: List[LayerSpec]
    final_norm: NormSpec
    tie_word_embeddings: bool
    max_positions: int
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    head_name: str = "lm_head.weight"
    run_order: List[RunEntry] = field(default_factory=list)
    # y = embedding * embedding_scale (1.0 for the reference's dense path,
    # src/model/dense.rs:1959-1967 gathers rows with no scaling)
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()

    def __post_init__(self) -> None:
        if not self.run_order:
            self.run_order = [RunEntry(i, i) for i in range(len(self.layers))]

    def cache_entries(self) -> Dict[int, int]:
        """cache entry -> the layer whose mixer defines its shape (the first
        run that writes it)."""
        out: Dict[int, int] = {}
        for run in self.run_order:
            if run.writes_cache and run.cache not in out:
                out[run.cache] = run.layer
        for run in self.run_order:
            if run.cache not in out:
                raise ValueError(
                    f"run order reads cache entry {run.cache} that no run writes"
                )
        return out


def names_dict(names: Tuple[Tuple[str, str], ...]) -> Dict[str, str]:
    return dict(names)
