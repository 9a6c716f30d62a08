from .tensor_spec import TensorSpec
from .safetensors_io import SafeTensorsError, load_file, parse, save_file, serialize
from .loader import WeightError, check_tensors, load_checkpoint, to_runtime_dtype
from .random_init import (random_tensors, random_tensors_on_device, standard_normal,
                          write_random_model)

__all__ = [
    "TensorSpec", "SafeTensorsError", "load_file", "parse", "save_file", "serialize",
    "WeightError", "check_tensors", "load_checkpoint", "to_runtime_dtype",
    "random_tensors", "random_tensors_on_device", "standard_normal", "write_random_model",
]
