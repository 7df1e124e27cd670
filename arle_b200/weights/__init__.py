from .loader import WeightError, kept_dtype, load_weights
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["WeightError", "kept_dtype", "load_weights", "random_tensors", "write_random_model", "SafetensorsError",
           "SafetensorsFile", "write_safetensors"]
