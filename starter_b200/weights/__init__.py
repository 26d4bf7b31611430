"""Weights: the safetensors container, the checked loader, and seeded random weights."""

from .loader import Checkpoint, WeightsError, check_tensors, expected_tensors
from .random_weights import RandomSource, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["Checkpoint", "WeightsError", "check_tensors", "expected_tensors", "RandomSource", "write_model_folder",
           "SafetensorsError", "SafetensorsFile", "write_safetensors"]
