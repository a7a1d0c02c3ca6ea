from .safetensors_io import Checkpoint, SafetensorsFile, write_safetensors  # noqa: F401
from .loader import check_names_and_shapes, load_model, load_spec, read_tensors  # noqa: F401
from .random_init import draw, random_model_on_device, random_tensors, write_random_model  # noqa: F401
