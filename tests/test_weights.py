"""Weights: file format, binding by name, errors, random mode (no GPU)."""

import json
import os
import struct

import numpy as np
import pytest
import torch

from reflex_b200 import CheckpointError, IoError
from reflex_b200.weights import (Checkpoint, SafetensorsFile, check_names_and_shapes, load_spec,
                                 read_tensors, write_random_model, write_safetensors)
from tiny_configs import TINY_A, TINY_B


def test_safetensors_roundtrip_keeps_element_types(tmp_path):
    t = {
        "a": torch.randn(3, 5).to(torch.bfloat16),
        "b": torch.randn(7),
        "c": torch.arange(6, dtype=torch.int64).reshape(2, 3),
        "d": torch.tensor(2.5),
        "e": torch.empty(0, 4),
    }
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t.items())
    f = SafetensorsFile(p)
    assert set(f.keys()) == set(t)
    for k, v in t.items():
        got = f.tensor(k)
        assert got.dtype == v.dtype and tuple(got.shape) == tuple(v.shape)
        assert torch.equal(got, v)
    f.close()


def test_file_is_readable_by_an_independent_reader(tmp_path):
    import plain_model

    d = write_random_model(TINY_A, 3, str(tmp_path / "m"), "bfloat16")
    mine = SafetensorsFile(os.path.join(d, "model.safetensors"))
    other = plain_model.read_safetensors(os.path.join(d, "model.safetensors"))
    assert set(mine.keys()) == set(other)
    for k in other:
        assert mine.tensor(k).dtype == torch.bfloat16
        np.testing.assert_array_equal(mine.tensor(k).double().numpy(), other[k])


def test_truncated_and_garbage_files(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x05")
    with pytest.raises(CheckpointError):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(CheckpointError):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(CheckpointError) as e:
        SafetensorsFile(str(p))
    assert "w" in str(e.value)
    with pytest.raises(IoError):
        Checkpoint(str(tmp_path / "nowhere"))


def _rewrite(folder, edit):
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {k: f.tensor(k).clone() for k in f.keys()}
    f.close()
    edit(tensors)
    write_safetensors(path, tensors.items())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_random_model(TINY_B, 1, str(tmp_path / "m"), "float32")

    def edit(t):
        del t["model.layers.1.self_attn.q_norm.weight"]
        del t["lm_head.weight"]
        t["model.layers.0.mlp.extra.weight"] = torch.zeros(2)
        t["model.layers.2.mlp.down_proj.weight"] = torch.zeros(5, 7)
        t["model.norm.weight"] = torch.zeros(95)

    _rewrite(d, edit)
    _, spec = load_spec(d)
    ck = Checkpoint(d)
    with pytest.raises(CheckpointError) as e:
        check_names_and_shapes(spec, ck)
    ck.close()
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.1.self_attn.q_norm.weight" in msg
    assert "lm_head.weight" in msg
    assert "unexpected tensors (1)" in msg and "model.layers.0.mlp.extra.weight" in msg
    assert "wrong shapes (2)" in msg
    assert "model.layers.2.mlp.down_proj.weight: expected [96, 320], found [5, 7]" in msg
    assert "model.norm.weight: expected [96], found [95]" in msg


def test_tied_model_needs_no_head_and_tolerates_one(tmp_path):
    d = write_random_model(TINY_A, 1, str(tmp_path / "m"), "float32")
    _, spec = load_spec(d)
    ck = Checkpoint(d)
    assert "lm_head.weight" not in ck
    check_names_and_shapes(spec, ck)
    ck.close()
    _rewrite(d, lambda t: t.__setitem__("lm_head.weight", t["model.embed_tokens.weight"].clone()))
    ck = Checkpoint(d)
    check_names_and_shapes(spec, ck)
    ck.close()


def test_stored_types_are_kept_on_the_host(tmp_path):
    d = write_random_model(TINY_A, 1, str(tmp_path / "m"), "bfloat16")
    _rewrite(d, lambda t: t.__setitem__("model.norm.weight", t["model.norm.weight"].float()))
    _, spec = load_spec(d)
    ck = Checkpoint(d)
    tensors = read_tensors(spec, ck)
    assert tensors["model.norm.weight"].dtype == torch.float32
    assert tensors["model.embed_tokens.weight"].dtype == torch.bfloat16
    ck.close()


def test_random_mode_is_a_function_of_config_and_seed(tmp_path):
    a = write_random_model(TINY_A, 5, str(tmp_path / "a"), "float32")
    b = write_random_model(TINY_A, 5, str(tmp_path / "b"), "float32")
    c = write_random_model(TINY_A, 6, str(tmp_path / "c"), "float32")
    fa, fb, fc = (SafetensorsFile(os.path.join(x, "model.safetensors")) for x in (a, b, c))
    differs = False
    for k in fa.keys():
        assert torch.equal(fa.tensor(k), fb.tensor(k))
        differs |= not torch.equal(fa.tensor(k), fc.tensor(k))
    assert differs
    w = fa.tensor("model.layers.0.mlp.up_proj.weight")
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    n = fa.tensor("model.layers.1.input_layernorm.weight")
    assert float(n.min()) >= 0.9 and float(n.max()) <= 1.1
    with open(os.path.join(a, "config.json")) as f:
        assert json.load(f)["hidden_size"] == TINY_A["hidden_size"]


def test_sharded_folder(tmp_path):
    d = write_random_model(TINY_A, 2, str(tmp_path / "m"), "float32")
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    names = f.keys()
    half = len(names) // 2
    parts = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    for fname, ns in parts.items():
        write_safetensors(os.path.join(d, fname), [(n, f.tensor(n).clone()) for n in ns])
    f.close()
    os.remove(os.path.join(d, "model.safetensors"))
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": {n: fname for fname, ns in parts.items() for n in ns}}, fh)
    _, spec = load_spec(d)
    ck = Checkpoint(d)
    check_names_and_shapes(spec, ck)
    assert len(read_tensors(spec, ck)) == len(names)
    ck.close()


def test_generation_config_adds_end_of_sequence_ids(tmp_path):
    """`generation_config.json`, when the folder has one, adds its
    end-of-sequence ids to config.json's; a malformed one is refused by name."""
    import json

    from reflex_b200 import InvalidInput
    from reflex_b200.weights.loader import load_spec
    from tiny_configs import TINY_A

    with open(tmp_path / "config.json", "w") as f:
        json.dump(dict(TINY_A, eos_token_id=7), f)
    assert load_spec(str(tmp_path))[1].eos_token_ids == (7,)
    with open(tmp_path / "generation_config.json", "w") as f:
        json.dump({"eos_token_id": [7, 9, 11], "temperature": 0.6}, f)
    assert load_spec(str(tmp_path))[1].eos_token_ids == (7, 9, 11)
    with open(tmp_path / "generation_config.json", "w") as f:
        json.dump({"eos_token_id": "seven"}, f)
    with pytest.raises(InvalidInput, match="generation_config.json"):
        load_spec(str(tmp_path))


def test_random_draw_is_a_function_of_seed_name_and_index():
    """N(0, 0.02) for matrices, 1 + U(-0.1, 0.1) for norms; the same values in one
    piece or in parts; other seeds and names give other values; bfloat16 is the
    32-bit draw rounded to nearest even."""
    from reflex_b200.weights.random_init import draw, draw_host, tensor_key

    x = draw("model.layers.0.mlp.up_proj.weight", (300, 1000), "matrix", 7).numpy()
    assert abs(float(x.mean())) < 2e-4 and abs(float(x.std()) - 0.02) < 2e-4
    assert 0.05 < float(np.abs(x).max()) < 0.12  # twelve uniforms: tails to six deviations at most
    frac = float((np.abs(x) < 0.02).mean())
    assert abs(frac - 0.6827) < 0.01
    w = draw("model.norm.weight", (5000,), "norm", 7).numpy()
    assert 0.9 < float(w.min()) < 0.905 and 1.095 < float(w.max()) < 1.1 and abs(float(w.mean()) - 1.0) < 3e-3
    key = tensor_key(7, "t")
    whole = draw_host(key, 1001, "normal", 0.0, 0.02)
    parts = np.concatenate([draw_host(key, 333, "normal", 0.0, 0.02), draw_host(key, 668, "normal", 0.0, 0.02, 333)])
    assert np.array_equal(whole, parts)
    assert not np.array_equal(whole, draw_host(tensor_key(8, "t"), 1001, "normal", 0.0, 0.02))
    assert not np.array_equal(whole, draw_host(tensor_key(7, "u"), 1001, "normal", 0.0, 0.02))
    b = draw("model.layers.0.mlp.up_proj.weight", (300, 1000), "matrix", 7, dtype=torch.bfloat16)
    assert torch.equal(b, torch.from_numpy(x).to(torch.bfloat16))
