from .errors import SafetensorsFormatError, WeightsMismatchError
from .safetensors_io import SafetensorsFile, write_safetensors
from .loader import TensorSpec, WeightSource, check_against, load_checked, storage_dtype
from .random_init import random_tensor, random_tensors, write_random_model

__all__ = [
    "SafetensorsFormatError", "WeightsMismatchError", "SafetensorsFile", "write_safetensors",
    "TensorSpec", "WeightSource", "check_against", "load_checked", "storage_dtype",
    "random_tensor", "random_tensors", "write_random_model",
]
