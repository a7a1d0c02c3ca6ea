"""Configuration and registry (no GPU)."""

import copy

import pytest

from reflex_b200 import CheckpointError, UnsupportedArchitecture
from reflex_b200 import models  # noqa: F401
from reflex_b200.config import Qwen3Config, resolve_architecture, spec_from_config_dict
from tiny_configs import ALL, TINY_A, TINY_B, TINY_C


def test_every_size_comes_from_config_json():
    for name, cfg in ALL.items():
        typed, spec = spec_from_config_dict(cfg)
        assert isinstance(typed, Qwen3Config)
        assert spec.vocab_size == cfg["vocab_size"]
        assert spec.hidden_size == cfg["hidden_size"]
        assert len(spec.layers) == cfg["num_hidden_layers"]
        assert spec.max_positions == cfg["max_position_embeddings"]
        assert spec.tie_word_embeddings == cfg["tie_word_embeddings"]
        for layer in spec.layers:
            m = layer.mixer
            assert (m.num_heads, m.num_kv_heads, m.head_dim) == (
                cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"])
            assert m.scale == pytest.approx(cfg["head_dim"] ** -0.5)
            assert m.position.theta == cfg["rope_theta"]
            assert m.position.rotary_dim == cfg["head_dim"]
            assert m.qk_norm.eps == cfg["rms_norm_eps"] == layer.mixer_norm.eps
            assert layer.feed_forward.intermediate_size == cfg["intermediate_size"]


def test_tiny_configs_differ_in_every_size():
    keys = ["num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
            "head_dim", "intermediate_size", "vocab_size", "rope_theta", "rms_norm_eps",
            "max_position_embeddings"]
    for k in keys:
        assert len({TINY_A[k], TINY_B[k], TINY_C[k]}) == 3 or k == "num_key_value_heads", k
    assert TINY_A["tie_word_embeddings"] != TINY_B["tie_word_embeddings"]


def test_registry_both_names_and_unknown():
    a = resolve_architecture({"architectures": ["Qwen3ForCausalLM"]})
    b = resolve_architecture({"model_type": "qwen3"})
    assert a is b
    with pytest.raises(UnsupportedArchitecture) as e:
        resolve_architecture({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    assert "LlamaForCausalLM" in str(e.value) and "qwen3" in str(e.value)


def test_missing_keys_are_listed_together():
    cfg = copy.deepcopy(TINY_A)
    del cfg["rms_norm_eps"], cfg["rope_theta"], cfg["vocab_size"]
    with pytest.raises(CheckpointError) as e:
        Qwen3Config.from_dict(cfg)
    for k in ("rms_norm_eps", "rope_theta", "vocab_size"):
        assert k in str(e.value)


def test_defaults_follow_the_reference():
    cfg = copy.deepcopy(TINY_A)
    del cfg["head_dim"], cfg["num_key_value_heads"]
    c = Qwen3Config.from_dict(cfg)
    assert c.head_dim == cfg["hidden_size"] // cfg["num_attention_heads"]
    assert c.num_key_value_heads == cfg["num_attention_heads"]


def test_rope_theta_in_rope_parameters():
    cfg = copy.deepcopy(TINY_A)
    theta = cfg.pop("rope_theta")
    cfg["rope_parameters"] = {"rope_theta": theta, "rope_type": "default"}
    assert Qwen3Config.from_dict(cfg).rope_theta == theta


@pytest.mark.parametrize("patch,needle", [
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"rope_parameters": {"rope_theta": 1e4, "rope_type": "linear", "factor": 2.0}}, "rope_scaling"),
    ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"mlp_bias": True}, "mlp_bias"),
])
def test_unsupported_options_are_rejected_by_name(patch, needle):
    cfg = copy.deepcopy(TINY_A)
    cfg.update(patch)
    with pytest.raises(UnsupportedArchitecture) as e:
        Qwen3Config.from_dict(cfg)
    assert needle in str(e.value)


@pytest.mark.parametrize("patch", [
    {"num_key_value_heads": 3}, {"head_dim": 15}, {"vocab_size": 0}, {"rms_norm_eps": 0.0},
    {"num_hidden_layers": -1}, {"layer_types": ["full_attention"]},
])
def test_bad_values(patch):
    cfg = copy.deepcopy(TINY_A)
    cfg.update(patch)
    with pytest.raises(CheckpointError):
        Qwen3Config.from_dict(cfg)


def test_sliding_layers_from_layer_types_and_from_max_window_layers():
    _, spec = spec_from_config_dict(TINY_C)
    assert [l.mixer.window for l in spec.layers] == [None, 37, None, 37]
    cfg = copy.deepcopy(TINY_C)
    del cfg["layer_types"]
    cfg["max_window_layers"] = 3
    _, spec = spec_from_config_dict(cfg)
    assert [l.mixer.window for l in spec.layers] == [None, None, None, 37]
    cfg["use_sliding_window"] = False
    _, spec = spec_from_config_dict(cfg)
    assert [l.mixer.window for l in spec.layers] == [None] * 4


def test_config_roundtrip():
    for cfg in ALL.values():
        c = Qwen3Config.from_dict(cfg)
        assert Qwen3Config.from_dict(c.to_dict()) == c


def test_run_order_defaults_and_cache_entries():
    _, spec = spec_from_config_dict(TINY_B)
    assert [(r.layer, r.cache, r.writes_cache) for r in spec.run_order] == [(i, i, True) for i in range(3)]
    assert spec.cache_entries() == {0: 0, 1: 1, 2: 2}


def test_run_time_switches_are_validated():
    """A bad value of an environment switch is an error that names it, not a
    silent default (the reference validates its own the same way:
    src/model/kernels.rs:244-259)."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for name, bad in (("REFLEX_B200_FUSE_NORM", "yes"), ("REFLEX_B200_DECODE_SPLITS", "many"),
                      ("REFLEX_B200_GEMV_MAX_ROWS", "4096")):
        env = dict(os.environ, **{name: bad})
        res = subprocess.run([sys.executable, "-c", "import reflex_b200.ops"], cwd=root, env=env,
                             capture_output=True, text=True)
        if name == "REFLEX_B200_DECODE_SPLITS":
            # read when a decode step picks its splits, not at import
            res = subprocess.run([sys.executable, "-c",
                                  "import reflex_b200.ops as o; o.decode_splits(1, 8, 8, 4)"],
                                 cwd=root, env=env, capture_output=True, text=True)
        assert res.returncode != 0 and "InvalidInput" in res.stderr and name in res.stderr, res.stderr


def test_weights_option_flag_then_environment_then_default(monkeypatch):
    """src/model/loading.rs:44-62: the flag wins, then REFLEX_WEIGHTS when set
    and not empty, then the caller's default; a bad value names its source."""
    from reflex_b200.api import EngineOptions, resolve_weights
    from reflex_b200.errors import InvalidInput

    monkeypatch.delenv("REFLEX_WEIGHTS", raising=False)
    assert resolve_weights() == "bf16"
    assert resolve_weights(default="f32") == "f32"
    assert resolve_weights("f32") == "f32"
    monkeypatch.setenv("REFLEX_WEIGHTS", "f32")
    assert resolve_weights() == "f32"
    assert resolve_weights("bf16") == "bf16"
    monkeypatch.setenv("REFLEX_WEIGHTS", "")
    assert resolve_weights() == "bf16"
    monkeypatch.setenv("REFLEX_WEIGHTS", "f8")
    with pytest.raises(InvalidInput) as e:
        resolve_weights()
    assert "REFLEX_WEIGHTS" in str(e.value)
    assert resolve_weights("f32") == "f32"  # a flag is not affected by a bad environment
    with pytest.raises(InvalidInput):
        resolve_weights("f16")
    o = EngineOptions()
    assert (o.weights, o.max_tokens, o.max_batch, o.use_graphs) == (None, 16384, 64, True)
