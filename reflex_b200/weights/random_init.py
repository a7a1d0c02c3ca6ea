"""Random weights from a configuration and a seed.

Linear and embedding weights are drawn N(0, 0.02), norm weights
1 + U(-0.1, 0.1).  Each tensor has a generator of its own, keyed by the seed
and the tensor's name, so any tensor can be drawn alone and the values do not
depend on the order of drawing.  `write_random_model` writes a model folder
(config.json, model.safetensors) that the loader reads like any other;
`random_tensors_on_device` draws straight into GPU memory for sizes where a
file would only cost time (the benchmark's).
The reference has no such mode: its fixtures are made outside the engine
(docs/DEVELOPMENT.md:362-369).
"""

from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Iterator, Tuple

import torch

from ..config.registry import spec_from_config_dict
from ..config.spec import ModelSpec
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def draw(name: str, shape, role: str, seed: int, device="cpu") -> torch.Tensor:
    """One float32 tensor."""
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    if role == "norm":
        return 1.0 + (torch.rand(shape, generator=g, device=device, dtype=torch.float32) * 0.2 - 0.1)
    return torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 0.02


def random_tensors(spec: ModelSpec, seed: int, dtype: torch.dtype, device="cpu") -> Iterator[Tuple[str, torch.Tensor]]:
    from ..engine.model import expected_tensors

    for name, (_where, info) in expected_tensors(spec).items():
        yield name, draw(name, info.shape, info.role, seed, device).to(dtype)


def write_random_model(config: Dict[str, Any], seed: int, out_dir: str, dtype: str = "bfloat16") -> str:
    """Write `out_dir/config.json` and `out_dir/model.safetensors`; returns
    `out_dir`.  `config` is a config.json dictionary of a registered
    architecture; `dtype` is the stored element type."""
    from .. import models  # noqa: F401

    torch_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    typed, spec = spec_from_config_dict(config)
    os.makedirs(out_dir, exist_ok=True)
    cfg = typed.to_dict() if hasattr(typed, "to_dict") else dict(config)
    cfg["torch_dtype"] = dtype
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=1)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), random_tensors(spec, seed, torch_dtype))
    return out_dir


def random_model_on_device(config: Dict[str, Any], seed: int, dtype: torch.dtype, device="cuda:0"):
    """A model with random weights drawn on the device, no file in between."""
    from .. import models  # noqa: F401
    from ..engine.model import CausalLM, expected_tensors

    _typed, spec = spec_from_config_dict(config)
    model = CausalLM(spec, dtype, device)
    store = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
    tensors = {}
    for name, (_where, info) in expected_tensors(spec).items():
        t = draw(name, info.shape, info.role, seed, device)
        tensors[name] = t if info.role == "norm" else t.to(store)
    model.bind(tensors)
    return model
