from .spec import (  # noqa: F401
    FeedForwardSpec,
    LayerSpec,
    MixerSpec,
    ModelSpec,
    NormSpec,
    PositionSpec,
    RunEntry,
)
from .registry import (  # noqa: F401
    Architecture,
    known_architectures,
    register_architecture,
    resolve_architecture,
    spec_from_config_dict,
)
from .qwen3 import Qwen3Config, read_config_json  # noqa: F401
