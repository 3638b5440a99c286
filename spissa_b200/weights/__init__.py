"""Safetensors in and out, the whole-checkpoint check, and random model folders."""
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
from .loader import TensorSource, WeightError, check_against, load_tensors
from .random_init import random_tensors, write_random_model

__all__ = ["SafetensorsError", "SafetensorsFile", "write_safetensors", "TensorSource", "WeightError",
           "check_against", "load_tensors", "random_tensors", "write_random_model"]
