"""Safetensors container, by-name loader and seeded random weights."""
from .loader import canonical_names, discover, inspect, load_tensors
from .random_init import random_tensors, write_model_folder
from .safetensors_io import CheckpointError, TensorEntry, read_header, read_tensor, write_file

__all__ = ["canonical_names", "discover", "inspect", "load_tensors", "random_tensors",
           "write_model_folder", "CheckpointError", "TensorEntry", "read_header",
           "read_tensor", "write_file"]
