"""reflex_b200: a small generation library for one GPU.

Everything between a request's token ids and its next token, for the
architectures registered under `reflex_b200.models`: typed configuration and a
registry, weights bound by name, layers put together from parts, a paged cache
with a slot per sequence, one step function, a generation loop with sampling,
and hand-written CUDA kernels for sm_100a.
"""

from .errors import (  # noqa: F401
    CacheError,
    CheckpointError,
    ContextOverflow,
    CudaError,
    InvalidInput,
    IoError,
    OutOfMemory,
    ReflexError,
    UnsupportedArchitecture,
)

__version__ = "0.1.0"


def load_model(model_dir, dtype="bfloat16", device="cuda:0"):
    """Read a model folder (config.json + safetensors) into a model on the GPU."""
    import torch

    from .weights.loader import load_model as _load

    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}.get(dtype, dtype)
    return _load(model_dir, dt, device)


from .sampling.params import SamplingParams  # noqa: E402,F401


def __getattr__(name):
    if name in ("Model", "EngineOptions", "System1Response", "System1CandidateResult", "resolve_weights"):
        from . import api

        return getattr(api, name)
    raise AttributeError(name)
