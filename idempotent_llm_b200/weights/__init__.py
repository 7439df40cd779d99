"""Safetensors reading/writing, loading by tensor name, random-weights mode."""

from .loader import TensorDecl, WeightError, load_weights, check_declared, storage_dtype
from .random_init import random_weights, write_random_model
from .safetensors_io import SafetensorsDir, SafetensorsFile, write_safetensors

__all__ = ["TensorDecl", "WeightError", "load_weights", "check_declared", "storage_dtype",
           "random_weights", "write_random_model", "SafetensorsDir", "SafetensorsFile", "write_safetensors"]
