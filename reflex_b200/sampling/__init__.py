from .params import SamplingParams, fresh_seed, uniform  # noqa: F401
from .sampler import Sampler  # noqa: F401
