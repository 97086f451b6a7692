"""Weights: safetensors files read and written by tensor name, and seeded random weights."""

from mini_engine_b200.weights.loader import WeightError, WeightSpec, load_weights
from mini_engine_b200.weights.random_init import random_tensors, write_random_model
from mini_engine_b200.weights.safetensors_io import SafetensorsFile, read_folder_index, write_safetensors

__all__ = [
    "SafetensorsFile",
    "WeightError",
    "WeightSpec",
    "load_weights",
    "random_tensors",
    "read_folder_index",
    "write_random_model",
    "write_safetensors",
]
