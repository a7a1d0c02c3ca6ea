"""One registry from an architecture's name to its model.

The reference dispatches on the checkpoint's architecture string
(src/model/mod.rs:800-826; accepted names src/model/config.rs:231-239).  Here
the string comes from config.json: `architectures[0]` (e.g. "Qwen3ForCausalLM")
or `model_type` (e.g. "qwen3"); both keys of an architecture point at the same
entry.  An entry has two functions: `parse(config dict) -> typed config` and
`build(typed config) -> ModelSpec`.  Adding an architecture is one
`register_architecture` call from a new module under `reflex_b200/models/`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, Tuple

from ..errors import UnsupportedArchitecture
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    parse: Callable[[Dict[str, Any]], Any]
    build: Callable[[Any], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(
    names: Iterable[str],
    parse: Callable[[Dict[str, Any]], Any],
    build: Callable[[Any], ModelSpec],
) -> Architecture:
    names = tuple(names)
    arch = Architecture(names[0], parse, build)
    for n in names:
        _ARCHITECTURES[n] = arch
    return arch


def known_architectures() -> Tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def resolve_architecture(cfg: Dict[str, Any]) -> Architecture:
    """The entry that config.json names, by `architectures` first and
    `model_type` second; unknown names are an error, never a fallthrough."""
    candidates = []
    archs = cfg.get("architectures")
    if isinstance(archs, (list, tuple)):
        candidates.extend(str(a) for a in archs)
    if cfg.get("model_type") is not None:
        candidates.append(str(cfg["model_type"]))
    for c in candidates:
        if c in _ARCHITECTURES:
            return _ARCHITECTURES[c]
    raise UnsupportedArchitecture(
        f"unsupported architecture {candidates!r}; known: {list(known_architectures())}"
    )


def spec_from_config_dict(cfg: Dict[str, Any]) -> Tuple[Any, ModelSpec]:
    arch = resolve_architecture(cfg)
    typed = arch.parse(cfg)
    return typed, arch.build(typed)
