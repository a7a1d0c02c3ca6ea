from .registry import (  # noqa: F401
    BLOCKS,
    FEED_FORWARDS,
    MIXERS,
    NORMS,
    POSITIONS,
    Rotation,
    TensorInfo,
    register_block,
    register_feed_forward,
    register_mixer,
    register_norm,
    register_position,
)
from . import norm, rope, mlp, attention, block  # noqa: F401,E402  (registers the parts)
