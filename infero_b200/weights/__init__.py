from .loader import WeightsError, check_names, convert, load_tensors
from .random_init import random_tensor, random_tensors, write_random_model
from .safetensors_io import SafetensorsDir, SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["WeightsError", "check_names", "convert", "load_tensors", "random_tensor", "random_tensors",
           "write_random_model", "SafetensorsDir", "SafetensorsError", "SafetensorsFile",
           "write_safetensors"]
