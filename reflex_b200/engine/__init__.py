from .batch import StepBatch, make_batch  # noqa: F401
from .model import CausalLM, RunContext, expected_tensors  # noqa: F401
from .step import Engine  # noqa: F401
