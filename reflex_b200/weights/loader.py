"""Binding a checkpoint's tensors to a model by name.

The reference binds GGUF tensors by name and reports a missing one with its
name (src/model/dense.rs:508-527, 648-650).  Here the names come from the
`ModelSpec`; the check runs over the whole model first and raises one error
that lists every missing tensor, every unexpected one and every wrong shape,
so a bad folder is diagnosed in one go.

Stored element types are kept: bfloat16 stays bfloat16 and 32-bit stays 32-bit
on the host (half precision is widened to 32-bit, which is exact; integer
tables become int32).  What precision a tensor is *used* in is the parts'
business: on the float32 path everything is widened to float32, on the
bfloat16 path matrices and tables are bfloat16 and norm weights float32.
"""

from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch

from ..config.qwen3 import read_config_json
from ..config.registry import spec_from_config_dict
from ..config.spec import ModelSpec
from ..errors import CheckpointError, InvalidInput
from .safetensors_io import Checkpoint


def _host_dtype(dtype: torch.dtype) -> torch.dtype:
    if dtype in (torch.bfloat16, torch.float32):
        return dtype
    if dtype in (torch.float16, torch.float64):
        return torch.float32
    if dtype in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool):
        return torch.int32
    return dtype


def check_names_and_shapes(spec: ModelSpec, ckpt) -> None:
    """Raise one `CheckpointError` naming everything that does not fit."""
    from ..engine.model import expected_tensors

    exp = expected_tensors(spec)
    have = set(ckpt.keys())
    optional_extra = set()
    if spec.tie_word_embeddings:
        optional_extra.add(spec.head_name)  # a tied model may still store its head
    missing = [n for n, (_, info) in exp.items() if n not in have and not info.optional]
    unexpected = sorted(have - set(exp) - optional_extra)
    wrong = []
    for n, (_, info) in exp.items():
        if n in have:
            dtype, shape = ckpt.info(n)
            if tuple(shape) != tuple(info.shape):
                wrong.append(f"{n}: expected {list(info.shape)}, found {list(shape)}")
            elif not (dtype.is_floating_point):
                wrong.append(f"{n}: expected a floating-point tensor, found {dtype}")
    if missing or unexpected or wrong:
        parts = [f"checkpoint does not match the '{spec.architecture}' model built from config.json:"]
        if missing:
            parts.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            parts.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            parts.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        raise CheckpointError("\n".join(parts))


def read_tensors(spec: ModelSpec, ckpt) -> Dict[str, torch.Tensor]:
    from ..engine.model import expected_tensors

    out = {}
    for name in expected_tensors(spec):
        if name in ckpt:
            t = ckpt.tensor(name)
            want = _host_dtype(t.dtype)
            out[name] = t if t.dtype == want else t.to(want)
    return out


def load_spec(model_dir: str) -> Tuple[object, ModelSpec]:
    from .. import models  # noqa: F401  (registers the architectures)

    typed, spec = spec_from_config_dict(read_config_json(model_dir))
    spec.eos_token_ids = merge_generation_config(model_dir, spec.eos_token_ids)
    return typed, spec


def merge_generation_config(model_dir: str, eos_ids) -> Tuple[int, ...]:
    """End-of-sequence ids of `generation_config.json`, when the folder has one,
    joined to config.json's (checkpoints often list further stop ids only
    there).  The reference takes its one end-of-sequence id from the tokenizer
    (src/sampling.rs:120-125); this library works on ids, so the model folder's
    json files are its only source."""
    import json
    import os

    path = os.path.join(model_dir, "generation_config.json")
    out = [int(e) for e in eos_ids]
    if os.path.isfile(path):
        try:
            with open(path) as f:
                eos = json.load(f).get("eos_token_id")
        except ValueError as e:
            raise InvalidInput(f"{path} is not valid JSON: {e}") from None
        if isinstance(eos, bool) or not (eos is None or isinstance(eos, (int, list, tuple))):
            raise InvalidInput(f"{path}: eos_token_id must be an integer or a list of integers")
        for e in ([] if eos is None else [eos] if isinstance(eos, int) else list(eos)):
            if isinstance(e, bool) or not isinstance(e, int) or e < 0:
                raise InvalidInput(f"{path}: eos_token_id must hold non-negative integers, got {e!r}")
            if e not in out:
                out.append(e)
    return tuple(out)


def load_model(model_dir: str, dtype: torch.dtype = torch.bfloat16, device="cuda:0"):
    """config.json -> registry -> ModelSpec -> parts -> weights bound by name."""
    from ..engine.model import CausalLM

    _typed, spec = load_spec(model_dir)
    ckpt = Checkpoint(model_dir)
    try:
        check_names_and_shapes(spec, ckpt)
        model = CausalLM(spec, dtype, device)
        tensors = read_tensors(spec, ckpt)
        if torch.device(device).type == "cuda":
            from .upload import upload_all

            tensors = upload_all(tensors, device)  # through pinned staging, element types kept
        model.bind(tensors)
    finally:
        ckpt.close()
    return model
