from .loader import WeightsError, expected_tensors, load_weights
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsFile, write_safetensors

__all__ = ["WeightsError", "expected_tensors", "load_weights", "random_tensors", "write_random_model",
           "SafetensorsFile", "write_safetensors"]
