"""Typed configuration of the Qwen3 dense architecture, read from config.json.

The reference reads the same quantities from GGUF metadata under the `qwen3.`
prefix (src/model/config.rs:177-364): `block_count`, `embedding_length`,
`attention.head_count`, `attention.head_count_kv`, `attention.key_length`,
`rope.freq_base`, `attention.layer_norm_rms_epsilon`, and the feed-forward
width from a tensor shape.  Here every one of them is a config.json key; no
size has a stand-in in code.  Defaults exist only where the reference has one
(src/model/config.rs:139-144, 312-314): `num_key_value_heads` defaults to the
number of query heads and `head_dim` to `hidden_size / num_attention_heads`.
Options the reference rejects for this architecture (RoPE scaling,
src/model/config.rs:273-289; bias tensors, src/model/config.rs:68-77) are
rejected here by name rather than ignored.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..errors import CheckpointError, UnsupportedArchitecture

REQUIRED_KEYS = (
    "vocab_size",
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "num_attention_heads",
    "rms_norm_eps",
    "max_position_embeddings",
)


@dataclass
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    # window of the sliding layers (query i sees key j iff 0 <= i-j < window),
    # and which layers slide; "full_attention" | "sliding_attention" per layer
    sliding_window: Optional[int] = None
    layer_types: List[str] = field(default_factory=list)
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    model_type: str = "qwen3"
    architectures: Tuple[str, ...] = ("Qwen3ForCausalLM",)

    def __post_init__(self) -> None:
        if not self.layer_types:
            self.layer_types = ["full_attention"] * self.num_hidden_layers
        self.validate()

    # ------------------------------------------------------------------
    def validate(self) -> None:
        def bad(msg: str) -> None:
            raise CheckpointError(f"config.json: {msg}")

        for key in (
            "vocab_size",
            "hidden_size",
            "intermediate_size",
            "num_hidden_layers",
            "num_attention_heads",
            "num_key_value_heads",
            "head_dim",
            "max_position_embeddings",
        ):
            value = getattr(self, key)
            if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
                bad(f"{key} must be a positive integer, got {value!r}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            bad(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})"
            )
        if self.head_dim % 2 != 0:
            bad(f"head_dim must be even for rotary pairs, got {self.head_dim}")
        if not (self.rms_norm_eps > 0.0):
            bad(f"rms_norm_eps must be positive, got {self.rms_norm_eps!r}")
        if not (self.rope_theta > 0.0):
            bad(f"rope_theta must be positive, got {self.rope_theta!r}")
        if len(self.layer_types) != self.num_hidden_layers:
            bad(
                f"layer_types has {len(self.layer_types)} entries for "
                f"{self.num_hidden_layers} layers"
            )
        for t in self.layer_types:
            if t not in ("full_attention", "sliding_attention"):
                raise UnsupportedArchitecture(f"config.json: unknown layer type {t!r}")
        if "sliding_attention" in self.layer_types:
            if not isinstance(self.sliding_window, int) or self.sliding_window <= 0:
                bad("sliding layers need a positive integer sliding_window")

    # ------------------------------------------------------------------
    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "Qwen3Config":
        missing = [k for k in REQUIRED_KEYS if k not in cfg or cfg[k] is None]
        rope_theta = cfg.get("rope_theta")
        rope_params = cfg.get("rope_parameters") or {}
        if rope_theta is None and isinstance(rope_params, dict):
            rope_theta = rope_params.get("rope_theta")
        if rope_theta is None:
            missing.append("rope_theta")
        if missing:
            raise CheckpointError(
                "config.json: missing required key(s): " + ", ".join(missing)
            )

        # rejected by name, never ignored
        scaling = cfg.get("rope_scaling")
        if scaling is None and isinstance(rope_params, dict):
            kind = rope_params.get("rope_type", rope_params.get("type", "default"))
            if kind not in (None, "default", "none"):
                scaling = rope_params
        if scaling is not None:
            kind = None
            if isinstance(scaling, dict):
                kind = scaling.get("rope_type", scaling.get("type"))
            if kind not in ("default", "none"):
                raise UnsupportedArchitecture(
                    f"config.json: rope_scaling {scaling!r} is not supported "
                    "(only unscaled rotary position encoding)"
                )
        if cfg.get("attention_bias", False):
            raise UnsupportedArchitecture(
                "config.json: attention_bias=true is not supported for qwen3"
            )
        act = cfg.get("hidden_act", "silu")
        if act != "silu":
            raise UnsupportedArchitecture(
                f"config.json: hidden_act {act!r} is not supported (only 'silu')"
            )
        if cfg.get("mlp_bias", False):
            raise UnsupportedArchitecture("config.json: mlp_bias=true is not supported")

        n_layers = cfg["num_hidden_layers"]
        n_heads = cfg["num_attention_heads"]
        n_kv = cfg.get("num_key_value_heads")
        if n_kv is None:
            n_kv = n_heads
        head_dim = cfg.get("head_dim")
        if head_dim is None:
            if not isinstance(n_heads, int) or n_heads <= 0 or cfg["hidden_size"] % n_heads:
                raise CheckpointError(
                    "config.json: head_dim is absent and hidden_size is not a "
                    "multiple of num_attention_heads"
                )
            head_dim = cfg["hidden_size"] // n_heads

        window = cfg.get("sliding_window")
        layer_types = cfg.get("layer_types")
        if layer_types is None:
            if cfg.get("use_sliding_window", False) and window is not None:
                first = cfg.get("max_window_layers", n_layers)
                layer_types = [
                    "sliding_attention" if i >= first else "full_attention"
                    for i in range(n_layers)
                ]
            else:
                layer_types = ["full_attention"] * n_layers
        layer_types = list(layer_types)
        if "sliding_attention" not in layer_types:
            window = None

        eos = cfg.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)

        archs = cfg.get("architectures") or ("Qwen3ForCausalLM",)
        return cls(
            vocab_size=cfg["vocab_size"],
            hidden_size=cfg["hidden_size"],
            intermediate_size=cfg["intermediate_size"],
            num_hidden_layers=n_layers,
            num_attention_heads=n_heads,
            num_key_value_heads=n_kv,
            head_dim=head_dim,
            rms_norm_eps=float(cfg["rms_norm_eps"]),
            rope_theta=float(rope_theta),
            max_position_embeddings=cfg["max_position_embeddings"],
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            sliding_window=window,
            layer_types=layer_types,
            torch_dtype=str(cfg.get("torch_dtype", cfg.get("dtype", "bfloat16"))),
            bos_token_id=cfg.get("bos_token_id"),
            eos_token_ids=eos_ids,
            model_type=str(cfg.get("model_type", "qwen3")),
            architectures=tuple(archs),
        )

    def to_dict(self) -> Dict[str, Any]:
        sliding = "sliding_attention" in self.layer_types
        out: Dict[str, Any] = {
            "architectures": list(self.architectures),
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "attention_bias": False,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "use_sliding_window": sliding,
            "sliding_window": self.sliding_window if sliding else None,
            "layer_types": list(self.layer_types),
            "torch_dtype": self.torch_dtype,
        }
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            out["eos_token_id"] = (
                self.eos_token_ids[0]
                if len(self.eos_token_ids) == 1
                else list(self.eos_token_ids)
            )
        return out


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            cfg = json.load(f)
    except FileNotFoundError as e:
        from ..errors import IoError

        raise IoError(f"{path}: no such file") from e
    except json.JSONDecodeError as e:
        raise CheckpointError(f"{path}: not valid JSON: {e}") from e
    if not isinstance(cfg, dict):
        raise CheckpointError(f"{path}: top level must be an object")
    return cfg
