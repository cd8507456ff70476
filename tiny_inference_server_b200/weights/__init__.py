from .loader import WeightError, check_tensors, load_weights, read_safetensors
from .random_init import random_tensors, write_random_model

__all__ = ["WeightError", "check_tensors", "load_weights", "read_safetensors", "random_tensors",
           "write_random_model"]
