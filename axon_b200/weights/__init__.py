"""Weights from safetensors by tensor name, and seeded random models."""

from .loader import (WeightsError, expected_tensors, load_weights, random_tensor, random_weights,
                     write_random_model)
from .safetensors_io import Checkpoint, SafetensorsError, SafetensorsFile, write_safetensors

__all__ = [
    "Checkpoint", "SafetensorsError", "SafetensorsFile", "WeightsError", "expected_tensors",
    "load_weights", "random_tensor", "random_weights", "write_random_model", "write_safetensors",
]
