"""Weights: safetensors files, binding by tensor name, seeded random weights."""
from .loader import (
    WeightLoadError,
    iterate_folder,
    load_model_weights,
    load_named_tensors,
    load_state_dict,
)
from .random_init import init_random_weights_, random_state_dict, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, weight_files, write_safetensors

__all__ = [
    "SafetensorsError",
    "SafetensorsFile",
    "WeightLoadError",
    "init_random_weights_",
    "iterate_folder",
    "load_model_weights",
    "load_named_tensors",
    "load_state_dict",
    "random_state_dict",
    "weight_files",
    "write_random_model",
    "write_safetensors",
]
