"""Typed errors with stable numeric codes.

The kinds and their numbers follow the reference's `ReflexErrorCode`
(src/error.rs:72-90): values never change meaning and new kinds are only
appended.  Kinds that belong to parts this library does not have (GGUF,
tokenizer, LoRA, grammar) keep their numbers but are never raised; the
checkpoint-format kind (1) is used for safetensors / config.json faults, which
is the role `Gguf` plays in the reference.
"""

from __future__ import annotations


class ReflexError(Exception):
    """Base class; `code` is the stable category number, `kind` its name."""

    code = 12
    kind = "other"


class CheckpointError(ReflexError):
    """Malformed model folder: bad config.json, bad safetensors header, tensors
    that are missing, unexpected or of the wrong shape (reference: `Gguf`)."""

    code = 1
    kind = "checkpoint"


class UnsupportedArchitecture(ReflexError):
    """A well-formed model this library cannot run: unknown architecture name,
    or a known one with an option it rejects (src/error.rs:24-26)."""

    code = 2
    kind = "unsupported_architecture"


class CudaError(ReflexError):
    """A kernel launch or CUDA call failed, the native library is missing, or
    the GPU is not one these kernels are compiled for (src/error.rs:27-29)."""

    code = 3
    kind = "cuda"


class OutOfMemory(ReflexError):
    """The cache has no free slot or page left, or a device allocation failed."""

    code = 5
    kind = "out_of_memory"


class ContextOverflow(ReflexError):
    """A sequence would pass the most positions its model or the cache allows.

    The message starts with the reference's stable prefix
    (src/limits.rs:33 `context length exceeded`)."""

    code = 7
    kind = "context_overflow"

    def __init__(self, requested: int, limit: int, what: str = "positions"):
        self.requested = requested
        self.limit = limit
        super().__init__(
            f"context length exceeded: {requested} {what} requested, limit is {limit}"
        )


class CacheError(ReflexError):
    """Misuse of the cache: a slot freed twice, an unknown slot, a sequence
    that is not live (reference: `KvCache`)."""

    code = 8
    kind = "kv_cache"


class IoError(ReflexError):
    code = 10
    kind = "io"


class InvalidInput(ReflexError):
    """The caller passed an invalid argument, e.g. `max_new_tokens == 0`, an
    empty prompt, a token id outside the vocabulary, a sampling parameter out of
    range (src/error.rs:55-57)."""

    code = 11
    kind = "invalid_input"


ERROR_CODES = {
    0: "ok",
    1: "checkpoint",
    2: "unsupported_architecture",
    3: "cuda",
    4: "cublas",
    5: "out_of_memory",
    6: "tokenizer",
    7: "context_overflow",
    8: "kv_cache",
    9: "lora",
    10: "io",
    11: "invalid_input",
    12: "other",
    13: "panic",
    14: "grammar_dead_end",
}
