"""Random weights from a configuration and a seed.

Linear and embedding weights are drawn N(0, 0.02), norm weights
1 + U(-0.1, 0.1).  A value is a function of (seed, tensor name, element index)
alone, computed the same way on the host and on the device, so any tensor, or
any part of one, can be drawn alone, and a model drawn on the GPU can be
rebuilt tensor by tensor on the CPU.  `write_random_model` writes a model folder
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


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of one tensor's draw."""
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little")


_GOLDEN = 0x9E3779B97F4A7C15
_M1, _M2 = 0xBF58476D1CE4E5B9, 0x94D049BB133111EB


def _mix64(key: int, c: "np.ndarray") -> "np.ndarray":
    """The splitmix64 finaliser of key + c * golden, on uint64 arrays (wrapping)."""
    import numpy as np

    z = np.uint64(key) + c * np.uint64(_GOLDEN)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(_M1)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(_M2)
    return z ^ (z >> np.uint64(31))


def draw_host(key: int, n: int, kind: str, a: float, b: float, first: int = 0) -> "np.ndarray":
    """Elements [first, first + n) of the draw keyed by `key`, float32: a function
    of (key, element index) alone, in integer and single IEEE double operations,
    the same ones `csrc/random_fill.cu` runs, so host and device give the same
    bits.  kind "normal": mean a, deviation b (twelve 16-bit uniforms summed);
    "uniform": in (a, b)."""
    import numpy as np

    with np.errstate(over="ignore"):
        e = np.arange(first, first + n, dtype=np.uint64)
        if kind == "normal":
            # the twelve 16-bit numbers summed in two 32-bit lanes of a word, folded at the end
            lanes = np.zeros(n, dtype=np.uint64)
            mask = np.uint64(0x0000FFFF0000FFFF)
            for j in range(3):
                h = _mix64(key, np.uint64(3) * e + np.uint64(j))
                lanes += (h & mask) + ((h >> np.uint64(16)) & mask)
            s = (lanes & np.uint64(0xFFFFFFFF)) + (lanes >> np.uint64(32))
            x = (s.astype(np.float64) - 393210.0) / 65536.0
            v = a + x * b
        elif kind == "uniform":
            u = _mix64(key, np.uint64(3) * e) >> np.uint64(40)
            t = (u.astype(np.float64) + 0.5) / 16777216.0
            v = a + (b - a) * t
        else:
            raise ValueError(f"kind must be normal or uniform, got {kind!r}")
    return v.astype(np.float32)


ROLE_DRAWS = {"norm": ("uniform", 0.9, 1.1)}  # every other role: N(0, 0.02)


def draw(name: str, shape, role: str, seed: int, device="cpu", dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """One tensor of the model `seed` names: linear and embedding weights
    N(0, 0.02), norm weights 1 + U(-0.1, 0.1); on the host or on the device, with
    the same bits.  bfloat16 is the 32-bit draw rounded to nearest even."""
    import numpy as np

    kind, a, b = ROLE_DRAWS.get(role, ("normal", 0.0, 0.02))
    key = tensor_key(seed, name)
    n = 1
    for d in shape:
        n *= int(d)
    if torch.device(device).type == "cuda":
        import ctypes

        from ..ops import dt_code, native

        out = torch.empty(tuple(shape), dtype=dtype, device=device)
        fn = native.lib().rfx_random_fill
        fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_ulonglong,
                       ctypes.c_int, ctypes.c_double, ctypes.c_double, ctypes.c_void_p]
        fn.restype = ctypes.c_int
        with torch.cuda.device(device):
            st = fn(out.data_ptr(), dt_code(dtype), n, 0, key, 0 if kind == "normal" else 1, a, b,
                    torch.cuda.current_stream().cuda_stream)
        native.check(st, "random_fill")
        return out
    if n >= (1 << 24) and torch.cuda.is_available():
        # a large tensor for the host: drawn on the GPU (the same bits) and copied
        return draw(name, shape, role, seed, "cuda", dtype).cpu()
    parts, step = [], 1 << 22  # in pieces: the intermediate arrays are 8 bytes an element
    for first in range(0, n, step):
        parts.append(draw_host(key, min(step, n - first), kind, a, b, first))
    flat = np.concatenate(parts) if len(parts) != 1 else parts[0]
    return torch.from_numpy(flat).reshape(tuple(shape)).to(dtype)


def random_tensors(spec: ModelSpec, seed: int, dtype: torch.dtype, device="cpu") -> Iterator[Tuple[str, torch.Tensor]]:
    from ..engine.model import expected_tensors

    for name, (_where, info) in expected_tensors(spec).items():
        yield name, draw(name, info.shape, info.role, seed, device, dtype)


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
        tensors[name] = draw(name, info.shape, info.role, seed, device,
                             torch.float32 if info.role == "norm" else store)
    model.bind(tensors)
    return model
