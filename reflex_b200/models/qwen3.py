"""Qwen3 dense as data: its typed config turned into a `ModelSpec`.

Layer order (src/model/dense.rs:1337-1431, 1469-1481): RMSNorm -> q/k/v
projections -> per-head q/k RMSNorm -> NeoX rotary -> cache write -> causal
grouped-query attention with scale 1/sqrt(head_dim) -> output projection ->
residual add -> RMSNorm -> gate/up -> silu(gate)*up -> down -> residual add;
then final RMSNorm -> lm_head (src/model/mod.rs:1191-1202).  All layers are
alike except that a layer may slide (its window from config.json).  Tensor
names are the checkpoint's; the right column of `*_NAMES` is the only place
they occur.
"""

from __future__ import annotations

import math

from ..config.qwen3 import Qwen3Config
from ..config.registry import register_architecture
from ..config.spec import (
    FeedForwardSpec,
    LayerSpec,
    MixerSpec,
    ModelSpec,
    NormSpec,
    PositionSpec,
)

ATTENTION_NAMES = (
    ("q_proj", "self_attn.q_proj.weight"),
    ("k_proj", "self_attn.k_proj.weight"),
    ("v_proj", "self_attn.v_proj.weight"),
    ("o_proj", "self_attn.o_proj.weight"),
    ("q_norm", "self_attn.q_norm.weight"),
    ("k_norm", "self_attn.k_norm.weight"),
)
MLP_NAMES = (
    ("gate_proj", "mlp.gate_proj.weight"),
    ("up_proj", "mlp.up_proj.weight"),
    ("down_proj", "mlp.down_proj.weight"),
)
BLOCK_NAMES = (
    ("mixer_norm", "input_layernorm.weight"),
    ("feed_forward_norm", "post_attention_layernorm.weight"),
)


def attention_scale(head_dim: int) -> float:
    """1 / sqrtf((float) head_dim), both steps in 32-bit as the reference computes
    it (src/model/kernels.rs:3385-3398), so that the kernels get the same bits."""
    import numpy as np

    return float(np.float32(1.0) / np.sqrt(np.float32(head_dim)))


def build_qwen3_spec(cfg: Qwen3Config) -> ModelSpec:
    eps = cfg.rms_norm_eps
    head_norm = NormSpec("rmsnorm", cfg.head_dim, eps)
    rope = PositionSpec(
        "rope_neox", head_dim=cfg.head_dim, rotary_dim=cfg.head_dim, theta=cfg.rope_theta
    )
    layers = []
    for i in range(cfg.num_hidden_layers):
        window = cfg.sliding_window if cfg.layer_types[i] == "sliding_attention" else None
        mixer = MixerSpec(
            "gqa_attention",
            hidden_size=cfg.hidden_size,
            num_heads=cfg.num_attention_heads,
            num_kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim,
            scale=attention_scale(cfg.head_dim),
            window=window,
            qk_norm=head_norm,
            position=rope,
            names=ATTENTION_NAMES,
        )
        ffn = FeedForwardSpec(
            "swiglu",
            hidden_size=cfg.hidden_size,
            intermediate_size=cfg.intermediate_size,
            names=MLP_NAMES,
        )
        layers.append(
            LayerSpec(
                block="prenorm",
                prefix=f"model.layers.{i}.",
                mixer=mixer,
                feed_forward=ffn,
                mixer_norm=NormSpec("rmsnorm", cfg.hidden_size, eps),
                feed_forward_norm=NormSpec("rmsnorm", cfg.hidden_size, eps),
                names=BLOCK_NAMES,
            )
        )
    return ModelSpec(
        architecture="qwen3",
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        layers=layers,
        final_norm=NormSpec("rmsnorm", cfg.hidden_size, eps),
        tie_word_embeddings=cfg.tie_word_embeddings,
        max_positions=cfg.max_position_embeddings,
        embedding_name="model.embed_tokens.weight",
        final_norm_name="model.norm.weight",
        head_name="lm_head.weight",
        bos_token_id=cfg.bos_token_id,
        eos_token_ids=cfg.eos_token_ids,
    )


QWEN3 = register_architecture(
    ("Qwen3ForCausalLM", "qwen3"), Qwen3Config.from_dict, build_qwen3_spec
)
