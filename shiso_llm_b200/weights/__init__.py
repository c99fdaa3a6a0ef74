"""Checkpoint access: the safetensors container, loading by name, random weights."""

from .loader import WeightError, load_weights, target_dtype, weight_files
from .random_init import random_device_tensors, random_tensors, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
from .spec import INDEX, MATRIX, NORMAL, ONES, VECTOR, ZEROS, TensorSpec

__all__ = [
    "INDEX", "MATRIX", "NORMAL", "ONES", "VECTOR", "ZEROS",
    "SafetensorsError", "SafetensorsFile", "TensorSpec", "WeightError",
    "load_weights", "random_device_tensors", "random_tensors", "target_dtype", "weight_files",
    "write_model_folder", "write_safetensors",
]
